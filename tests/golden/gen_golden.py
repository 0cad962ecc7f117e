"""Regenerates the golden fixtures in this directory from the CPU checker (oracle/).

The reference itself cannot run where this is built (no JS runtime, no clang) and ships no golden vectors for the
Llama path, so these files are the checker's own outputs on the seeded workloads: they pin the checker against
accidental change and let GPU tests compare full-size runs without re-running minutes of CPU work.

  python tests/golden/gen_golden.py            # tiny + C1 (about half a minute on 8 cores)

Files:
  tiny_fp16.npz / tiny_int8.npz : dim 256, 2 layers, 4 heads, 2 kv heads (head_dim 64), vocab 1024 — ids, full logits
  c1_llama32_1b.npz             : Llama-3.2-1B architecture, 32-token prompt, 64 greedy tokens — ids, top-2 margins,
                                  max logit and the logits at 256 fixed vocabulary positions per step
  c1_llama32_1b_seed42.npz      : the same workload with prompt seed 42, whose greedy trajectory passes through
                                  positions where the two best fp16 logits are one unit in the last place apart

Prompt seed of the C1 fixture: with N(0, 0.02) random weights the two largest of 128256 fp16 logits are often within a
few units in the last place, where any reordering of an fp32 sum can change the greedy pick.  Token-exact comparison is
only meaningful on a trajectory that does not pass through such ties, so the fixture uses the first seed >= 42 whose
64 greedy steps all keep a top-1/top-2 margin of at least 3 fp16 units in the last place (C1_PROMPT_SEED, found by
running this checker over seeds 42, 43, ...).  The seed-42 trajectory is kept to test exactly that sensitivity.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.util import build_oracle, oracle_greedy  # noqa: E402
from denograd_b200 import synth  # noqa: E402
from denograd_b200.llama3 import MODEL_PARAMS  # noqa: E402

TINY = {"dim": 256, "n_heads": 4, "n_kv_heads": 2, "n_layers": 2, "norm_eps": 1e-5, "rope_theta": 500000,
        "vocab_size": 1024, "hidden_dim": 512}
C1_SAMPLE = np.linspace(0, 128255, 256).astype(np.int64)
C1_PROMPT_SEED = 52


def tiny(int8: bool) -> None:
    m = build_oracle(TINY, max_context=64, max_batch=2, int8=int8, tied=True)
    prompt = synth.prompt_tokens(8, TINY["vocab_size"], batch=2)
    ids, logits, margins = oracle_greedy(m, prompt, 12)
    np.savez_compressed(os.path.join(HERE, f"tiny_{'int8' if int8 else 'fp16'}.npz"), prompt=prompt, ids=ids,
                        logits=logits.astype(np.float16), margins=margins.astype(np.float32))


def c1() -> None:
    p = dict(MODEL_PARAMS["1B"]["args"])
    for seed, name in ((C1_PROMPT_SEED, "c1_llama32_1b.npz"), (42, "c1_llama32_1b_seed42.npz")):
        m = build_oracle(p, max_context=128, max_batch=1, int8=False, tied=True)
        prompt = synth.prompt_tokens(32, p["vocab_size"], seed=seed)
        ids, logits, margins = oracle_greedy(m, prompt, 64)
        top = logits.max(axis=2)
        np.savez_compressed(os.path.join(HERE, name), prompt=prompt, prompt_seed=np.int64(seed), ids=ids,
                            margins=margins.astype(np.float32), max_logit=top.astype(np.float32),
                            margin_ulps=(margins / 2.0 ** (np.floor(np.log2(np.abs(top))) - 10)).astype(np.float32),
                            sample_idx=C1_SAMPLE, sample_logits=logits[:, :, C1_SAMPLE].astype(np.float16))
        m.close()


if __name__ == "__main__":
    tiny(False)
    tiny(True)
    if "--no-c1" not in sys.argv:
        c1()
