"""Shared helpers of the test-suite: build the CPU checker's model with the same seeded tensors the device fills."""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402
from denograd_b200 import synth  # noqa: E402

LAYER_TENSORS = [  # (state-dict suffix, oracle id, rows, cols) filled in per config
    ("attention.wq", O.WQ), ("attention.wk", O.WK), ("attention.wv", O.WV), ("attention.wo", O.WO),
    ("feed_forward.w1", O.W1), ("feed_forward.w2", O.W2), ("feed_forward.w3", O.W3),
]


def tensor_shapes(p: dict) -> dict[str, tuple[int, int]]:
    d, hd = p["dim"], p["dim"] // p["n_heads"]
    kv, f = p["n_kv_heads"] * hd, p["hidden_dim"]
    return {"attention.wq": (d, d), "attention.wk": (kv, d), "attention.wv": (kv, d), "attention.wo": (d, d),
            "feed_forward.w1": (f, d), "feed_forward.w2": (d, f), "feed_forward.w3": (f, d)}


def synth_weight(name: str, shape, int8: bool, seed: int = synth.BASE_SEED):
    """(weight, scale-or-None) exactly as denograd_b200.synth.fill_tensor produces them on the device."""
    n = int(np.prod(shape))
    if int8:
        w = O.synth_uniform_i8(synth.name_seed(name + ".weight", seed), n).reshape(shape)
        s = O.synth_scale_f16(synth.name_seed(name + ".scale", seed), shape[0], synth.INT8_SCALE_BASE)
        return w, s
    return O.synth_normal_f16(synth.name_seed(name + ".weight", seed), n, synth.WEIGHT_STD).reshape(shape), None


def build_oracle(p: dict, max_context: int, max_batch: int = 1, int8: bool = False, tied: bool = True,
                 seed: int = synth.BASE_SEED) -> O.OracleModel:
    """Oracle model for architecture dict `p` (MODEL_PARAMS[...]['args'] layout) with the seeded synthetic weights."""
    cfg = O.OracleConfig(dim=p["dim"], n_layers=p["n_layers"], n_heads=p["n_heads"], n_kv_heads=p["n_kv_heads"],
                         hidden=p["hidden_dim"], vocab=p["vocab_size"], max_context=max_context, max_batch=max_batch,
                         quant=int(int8), quant_embed=int(int8), eps=p["norm_eps"], theta=float(p["rope_theta"]))
    m = O.OracleModel(cfg)
    shapes = tensor_shapes(p)
    ones = np.ones((p["dim"],), np.float16)
    for l in range(p["n_layers"]):
        for suffix, wid in LAYER_TENSORS:
            w, s = synth_weight(f"layers.{l}.{suffix}", shapes[suffix], int8, seed)
            m.set_weight(l, wid, w, s)
        m.set_weight(l, O.ATTN_NORM, ones)
        m.set_weight(l, O.FFN_NORM, ones)
    emb, emb_s = synth_weight("tok_embeddings", (p["vocab_size"], p["dim"]), int8, seed)
    m.set_weight(-1, O.TOK_EMB, emb, emb_s)
    if tied:
        m.set_weight(-1, O.OUTPUT, emb, emb_s)
    else:
        out, out_s = synth_weight("output", (p["vocab_size"], p["dim"]), int8, seed)
        m.set_weight(-1, O.OUTPUT, out, out_s)
    m.set_weight(-1, O.NORM, ones)
    return m


def oracle_greedy(m: O.OracleModel, prompt: np.ndarray, n_new: int):
    """Token-at-a-time prefill then greedy decode, as Llama3._prefill / chat do.  Returns (ids [B,n_new],
    logits of every generated position [n_new,B,V] as fp32, top1-top2 margins [n_new,B])."""
    prompt = np.asarray(prompt, np.int32)
    B, P = prompt.shape
    pos = 0
    logits = nxt = None
    for i in range(P):
        logits, nxt = m.forward(prompt[:, i:i + 1], pos)
        pos += 1
    ids = np.empty((B, n_new), np.int32)
    all_logits, margins = [], []
    for i in range(n_new):
        ids[:, i] = nxt
        all_logits.append(logits.copy())
        top2 = np.partition(logits, -2, axis=1)[:, -2:]
        margins.append(top2[:, 1] - top2[:, 0])
        if i + 1 < n_new:
            logits, nxt = m.forward(nxt.reshape(B, 1), pos)
            pos += 1
    return ids, np.stack(all_logits), np.stack(margins)


# A shape the single-kernel decode step is instantiated for when it is cut in two by tensor parallelism (per rank: 4
# query heads of 64 on 1 kv head, 6656 hidden columns = four rows per 64 KB pass, as the 1B model's 8192) and whose
# vocabulary shard (501 rows) does not divide by the number of CTAs.
TP_STEP_ARCH = {"dim": 512, "n_heads": 8, "n_kv_heads": 2, "n_layers": 3, "norm_eps": 1e-5, "rope_theta": 500000,
                "vocab_size": 1002, "hidden_dim": 13312}
