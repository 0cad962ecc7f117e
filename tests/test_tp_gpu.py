"""Tensor parallelism on real GPUs: 2 ranks (processes), all-reduce after wo and w2 (the peer-memory kernel, and NCCL
alone), sharded vocabulary.  Skipped when fewer than 2 GPUs are visible.  NVLS is switched off for the test processes
(plain ring/tree NCCL); the peer-memory kernel uses plain loads and stores."""
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from denograd_b200 import ffi, synth
from tests.golden.gen_golden import TINY
from tests.util import ROOT, TP_STEP_ARCH, build_oracle, oracle_greedy

pytestmark = pytest.mark.gpu


def _gpu_count() -> int:
    n = ctypes.c_int32(0)
    try:
        return n.value if ffi.load().jg_device_count(ctypes.byref(n)) == 0 else 0
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("peer,quant,arch", [("1", "float16", "tiny"), ("0", "float16", "tiny"), ("1", "int8", "tiny"),
                                             ("1", "float16", "step")])
def test_two_rank_tensor_parallel_matches_the_checker(peer, quant, arch):
    """`step`: a shape whose decode step runs as the single persistent kernel, with the exchanges inside it."""
    batch, n_new, world = 2, 8, 2
    P = TP_STEP_ARCH if arch == "step" else TINY
    with tempfile.TemporaryDirectory() as work:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", JG_TP_PEER=peer, JG_PEER_TIMEOUT_MS="5000", JG_TEST_ARCH=arch)
        logs = [open(os.path.join(work, f"rank{r}.log"), "w+") for r in range(world)]
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "tp_worker.py"), str(r), str(world), work,
                                   str(batch), str(n_new), quant], env=env, stdout=logs[r], stderr=subprocess.STDOUT)
                 for r in range(world)]
        for p in procs:
            p.wait(timeout=400)  # a stuck rank ends itself after 150 s (see tp_worker.py)
        outs = []
        for f in logs:
            f.seek(0)
            outs.append(f.read())
            f.close()
        assert all(p.returncode == 0 for p in procs), "\n".join(outs)[-4000:]
        res = [np.load(os.path.join(work, f"out_{r}.npz")) for r in range(world)]
        if peer == "1":  # the peer-memory path must really have been the one that ran
            assert all(open(os.path.join(work, f"peer_{r}.txt")).read() == "1" for r in range(world)), "peer memory not mapped"
        took_step = [open(os.path.join(work, f"step_{r}.txt")).read() == "1" for r in range(world)]
        assert took_step == [arch == "step"] * world, took_step
    m = build_oracle(P, max_context=64, max_batch=batch, int8=(quant == "int8"), tied=True)
    prompt = synth.prompt_tokens(6, P["vocab_size"], batch=batch, seed=31)
    ref_ids, ref_logits, margins = oracle_greedy(m, prompt, n_new)
    Vl = P["vocab_size"] // world
    for r in range(world):
        assert int(res[r]["offset"]) == r * Vl
        assert (res[r]["ids"] == res[0]["ids"]).all() and (res[r]["loop"] == res[0]["ids"]).all()
        assert np.abs(res[r]["logits"] - ref_logits[-1][:, r * Vl:(r + 1) * Vl]).max() <= 2e-2
    ulp = 2.0 ** (np.floor(np.log2(np.abs(ref_logits.max(axis=2)))) - 10)
    safe = (margins / ulp) >= 3
    for b in range(batch):
        n = n_new if safe[:, b].all() else int(np.argmin(safe[:, b]))
        assert (res[0]["ids"][b, :n] == ref_ids[b, :n]).all()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs 2 GPUs")
def test_a_peer_that_never_joins_is_reported_not_waited_for():
    """Host-made failure (a rank stops launching between steps, nothing in flight): the waiting rank's kernel gives up
    after JG_PEER_TIMEOUT_MS, the next synchronisation returns JG_ETIMEDOUT (110) and the device remains usable."""
    world = 2
    with tempfile.TemporaryDirectory() as work:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", JG_TP_PEER="1", JG_PEER_TIMEOUT_MS="1000")
        logs = [open(os.path.join(work, f"rank{r}.log"), "w+") for r in range(world)]
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "tp_worker.py"), str(r), str(world), work,
                                   "1", "1", "missing-peer"], env=env, stdout=logs[r], stderr=subprocess.STDOUT)
                 for r in range(world)]
        for p in procs:
            p.wait(timeout=300)
        outs = []
        for f in logs:
            f.seek(0)
            outs.append(f.read())
            f.close()
        assert all(p.returncode == 0 for p in procs), "\n".join(outs)[-4000:]
        res = [np.load(os.path.join(work, f"out_{r}.npz")) for r in range(world)]
    assert bool(res[0]["ok_first"]) and bool(res[1]["ok_first"])
    assert int(res[0]["status"]) == 110 and bool(res[0]["usable"])
