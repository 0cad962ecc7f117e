"""CPU checks of the tensor-parallel host logic with two real ranks over gloo: the shard plan's windows recombine to
the unsharded layer (column-parallel outputs concatenate, row-parallel partial sums all-reduce), and the packed greedy
keys of a vocabulary-sharded output layer reduce to the lowest-index maximum."""
import os
import sys
import tempfile

import numpy as np
import pytest

from denograd_b200.multi import shard_plan
from tests.golden.gen_golden import TINY
from tests.util import ROOT


def test_shard_plan_covers_every_tensor_exactly_once():
    p = dict(TINY)
    d, hd = p["dim"], p["dim"] // p["n_heads"]
    world = 2
    plans = [shard_plan(p, r, world, tied=True) for r in range(world)]
    for name, sh0 in plans[0].items():
        rows = sum(pl[name].rows for pl in plans) if sh0.cols == sh0.cols_full else sh0.rows
        cols = sum(pl[name].cols for pl in plans) if sh0.cols != sh0.cols_full else sh0.cols
        if name.endswith("wq.weight") or name.endswith("wo.weight"):
            assert (rows, cols) == (d, d)
        if name.endswith("wk.weight"):
            assert (rows, cols) == (p["n_kv_heads"] * hd, d)
        if name.endswith("w2.weight"):
            assert (rows, cols) == (d, p["hidden_dim"])
        if name == "output.weight":
            assert (rows, cols) == (p["vocab_size"], d) and sh0.seed_name == "tok_embeddings.weight"
        # windows of different ranks are disjoint and adjacent
        assert plans[1][name].row0 == sh0.row0 + (sh0.rows if sh0.cols == sh0.cols_full else 0)
        assert plans[1][name].col0 == sh0.col0 + (sh0.cols if sh0.cols != sh0.cols_full else 0)
    with pytest.raises(ValueError):
        shard_plan(p, 0, 3, tied=True)


def test_int8_shard_plan_carries_the_scales_with_the_rows():
    """Per-output-row scales follow the rows of their weight's window: split with column-parallel weights,
    whole (replicated) with the row-parallel wo / w2, whose windows span every output row."""
    p = dict(TINY)
    d = p["dim"]
    plans = [shard_plan(p, r, 2, tied=True, int8=True) for r in range(2)]
    for r, plan in enumerate(plans):
        for name, sh in plan.items():
            if not name.endswith(".weight"):
                continue
            sc = plan[name.replace(".weight", ".scale")]
            assert (sc.rows, sc.cols, sc.row0, sc.col0) == (sh.rows, 1, sh.row0, 0), name
            assert sc.seed_name == sh.seed_name.replace(".weight", ".scale")
        assert plan["layers.0.attention.wo.scale"].rows == d and plan["layers.0.attention.wo.scale"].row0 == 0
        assert plan["layers.0.feed_forward.w1.scale"].row0 == r * (p["hidden_dim"] // 2)
        assert plan["output.scale"].seed_name == "tok_embeddings.scale"
    assert not any(k.endswith(".scale") for k in shard_plan(p, 0, 2, tied=True))


def _rank(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    from tests.util import synth_weight, tensor_shapes
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = dict(TINY)
    plan = shard_plan(p, rank, world, tied=True)
    shapes = tensor_shapes(p)
    full = {k: synth_weight(f"layers.0.{k}", shapes[k], False)[0] for k in shapes}

    def win(name):
        sh = plan[f"layers.0.{name}.weight"]
        return np.ascontiguousarray(full[name][sh.row0:sh.row0 + sh.rows, sh.col0:sh.col0 + sh.cols])

    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, p["dim"])).astype(np.float16)
    # column-parallel: each rank's rows of w1 give its slice of the output
    y_local = O.linear_f16(x, win("feed_forward.w1"))
    gathered = [torch.zeros(y_local.shape, dtype=torch.float16) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(y_local))
    y = np.concatenate([g.numpy() for g in gathered], axis=1)
    # row-parallel: fp32 partial sums over this rank's K-slice, all-reduced, rounded once
    w2 = win("feed_forward.w2")
    sh = plan["layers.0.feed_forward.w2.weight"]
    part = y[:, sh.col0:sh.col0 + sh.cols].astype(np.float32) @ w2.astype(np.float32).T
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    z = t.numpy().astype(np.float16)
    # greedy keys: (ordered fp16 value << 32) | ~global index, reduced with max
    Vl = p["vocab_size"] // world
    logits = np.zeros(Vl, np.float16)
    logits[5] = 3.0 if rank == 1 else 1.0
    logits[9] = 3.0  # rank 0's index 9 ties with rank 1's index Vl + 5: the lower global index must win
    u = logits.view(np.uint16).astype(np.int64)
    okey = np.where(u & 0x8000, (~u) & 0xFFFF, u | 0x8000)
    key = (okey << 32) | (0xFFFFFFFF - (np.arange(Vl) + rank * Vl))
    k = torch.tensor([int(key.max())], dtype=torch.int64)
    dist.all_reduce(k, op=dist.ReduceOp.MAX)
    if rank == 0:
        np.savez(os.path.join(out_dir, "r0.npz"), y=y, z=z, tok=0xFFFFFFFF - (int(k.item()) & 0xFFFFFFFF),
                 y_ref=O.linear_f16(x, full["feed_forward.w1"]), z_ref=O.linear_f16(O.linear_f16(x, full["feed_forward.w1"]), full["feed_forward.w2"]))
    dist.destroy_process_group()


def test_two_ranks_recombine_to_the_unsharded_layer():
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    with tempfile.TemporaryDirectory() as out_dir:
        mp.spawn(_rank, args=(2, port, out_dir), nprocs=2, join=True)
        r = np.load(os.path.join(out_dir, "r0.npz"))
        assert (r["y"] == r["y_ref"]).all()  # column-parallel slices are the unsharded outputs, bit for bit
        d = np.abs(r["z"].astype(np.float32) - r["z_ref"].astype(np.float32))
        assert d.max() <= 2e-3 * max(1.0, np.abs(r["z_ref"].astype(np.float32)).max())  # summation order only
        assert int(r["tok"]) == 9
