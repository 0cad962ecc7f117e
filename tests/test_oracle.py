"""CPU checks of the checker itself.  The reference holds no golden vectors for the Llama path (parity unpinned),
so the restatement is pinned by (i) known answers that follow from the reference source, (ii) an independent numpy
float64 implementation of the same model, (iii) the committed fixtures in tests/golden (its own earlier outputs)."""
import math
import os

import numpy as np
import pytest

from denograd_b200 import synth
from denograd_b200.nn import Int8Linear
from oracle import oracle as O
from tests.golden.gen_golden import TINY
from tests.util import ROOT, build_oracle, oracle_greedy, synth_weight, tensor_shapes

GOLD = os.path.join(ROOT, "tests", "golden")


# ------------------------------------------------------------------------------------------------ known answers
def test_xexp2_known_values():
    assert O.xexp2_f32(0.0) == 1.0 and O.xexp2_f32(1.0) == 2.0 and O.xexp2_f32(-3.0) == 0.125
    assert O.xexp2_f32(float("-inf")) == 0.0 and O.xexp2_f32(200.0) == float("inf")
    assert math.isnan(O.xexp2_f32(float("nan")))
    assert float(O.xexp2_f16(np.float16(0))) == 1.0 and float(O.xexp2_f16(np.float16(-23))) == 0.0
    assert np.isinf(O.xexp2_f16(np.float16(23.0)))


def test_xexp2_within_one_ulp_of_exp2():
    for x in np.linspace(-30, 30, 1501, dtype=np.float32):
        ref = 2.0 ** np.float64(x)
        assert abs(O.xexp2_f32(x) - ref) <= 1.2 * np.spacing(np.float32(ref)), x


def test_xsin_both_reductions():
    # below 30 the Cody-Waite branch runs, from 30 up the Payne-Hanek branch (rope angles reach 2*max_context)
    xs = np.concatenate([np.linspace(-29.9, 29.9, 801), np.linspace(30, 20000, 801)]).astype(np.float32)
    err = max(abs(O.xsin_f32(x) - math.sin(float(x))) for x in xs)
    assert err < 3e-7, err
    assert O.xsin_f32(0.0) == 0.0 and math.isnan(O.xsin_f32(float("inf")))


def test_freqs_cis_table():
    t = O.freqs_cis(64, 300, 500000.0).astype(np.float64)
    assert (t[0, :, 0] == 1.0).all() and (t[0, :, 1] == 0.0).all()  # position 0: cos 1, sin 0
    i = np.arange(32)
    ang = np.outer(np.arange(300), 1.0 / 500000.0 ** (2 * i / 64))
    assert np.abs(t[..., 0] - np.cos(ang)).max() < 6e-4 and np.abs(t[..., 1] - np.sin(ang)).max() < 6e-4


def test_rope_position_zero_is_identity_and_pairs_are_interleaved():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 4, 64)).astype(np.float16)
    t = O.freqs_cis(64, 16, 500000.0)
    assert (O.rope(x, t, [0, 0]) == x).all()
    y = O.rope(x, t, [5, 9]).astype(np.float64)
    for r, p in enumerate((5, 9)):
        c, s = t[p, :, 0].astype(np.float64), t[p, :, 1].astype(np.float64)
        a, b = x[r, :, 0::2].astype(np.float64), x[r, :, 1::2].astype(np.float64)
        assert np.abs(y[r, :, 0::2] - (a * c - b * s)).max() < 4e-3
        assert np.abs(y[r, :, 1::2] - (a * s + b * c)).max() < 4e-3


def test_argmax_lowest_index_among_ties():
    x = np.zeros(1000, np.float16)
    x[[17, 400, 999]] = 3.5
    assert O.argmax_f16(x) == 17
    assert O.argmax_f16(np.full(8, -2.0, np.float16)) == 0


def test_linear_is_fp32_accumulate_single_rounding():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 512)).astype(np.float16)
    w = (rng.standard_normal((40, 512)) * 0.05).astype(np.float16)
    y = O.linear_f16(x, w)
    acc = np.zeros((3, 40), np.float32)
    for k in range(512):  # strict ascending-k fp32 accumulation of exact products
        acc = acc + x[:, k:k + 1].astype(np.float32) * w[:, k].astype(np.float32)[None, :]
    assert (y == acc.astype(np.float16)).all()


def test_int8_linear_dequant_scheme_and_quantize_roundtrip():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((24, 256)) * 0.02).astype(np.float16)
    wq, s = O.quantize_w8(w)
    # half a step of rounding, plus the fp16 roundings of 1/scale and of W * (1/scale) near |q| = 127
    err = np.abs(w.astype(np.float32) - wq.astype(np.float32) * s.astype(np.float32)[:, None])
    assert (err <= 0.65 * s.astype(np.float32)[:, None]).all()
    host = Int8Linear.quantize({"layers.0.attention.wq.weight": w})
    assert (host["layers.0.attention.wq.weight"] == wq).all() and (host["layers.0.attention.wq.scale"] == s).all()
    x = rng.standard_normal((2, 256)).astype(np.float16)
    deq = (wq.astype(np.float16) * s[:, None]).astype(np.float16)  # half(Wq) * scale, rounded once
    assert (O.linear_w8(x, wq, s) == O.linear_f16(x, deq)).all()
    tok = np.array([3, 0, 23], np.int32)
    assert (O.embed_w8(tok, wq, s) == deq[tok]).all()


def test_repeat_kv_head_mapping_and_softmax():
    """Query head h must read kv head h // n_rep; with one cached position the output is exactly v."""
    rng = np.random.default_rng(3)
    H, G, hd = 8, 2, 64
    q = rng.standard_normal((1, 1, H, hd)).astype(np.float16)
    k = rng.standard_normal((1, 4, G, hd)).astype(np.float16)
    v = rng.standard_normal((1, 4, G, hd)).astype(np.float16)
    out = O.attention(q, k, v, 0).reshape(H, hd)
    for h in range(H):
        assert (out[h] == v[0, 0, h // (H // G)]).all()
    out = O.attention(q, k, v, 3).reshape(H, hd).astype(np.float64)
    for h in range(H):
        g = h // (H // G)
        s = (q[0, 0, h].astype(np.float64) @ k[0, :, g].astype(np.float64).T) / math.sqrt(hd)
        p = np.exp(s - s.max()); p /= p.sum()
        assert np.abs(out[h] - p @ v[0, :, g].astype(np.float64)).max() < 3e-3


def test_swiglu_matches_float64():
    g = np.linspace(-12, 12, 2001).astype(np.float16)
    u = np.full_like(g, 1.5)
    ref = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * 1.5
    got = O.swiglu(g, u).astype(np.float64)
    assert np.abs(got - ref).max() <= 0.012 * np.abs(ref).max()
    assert O.swiglu(np.array([-30.0], np.float16), np.array([1.0], np.float16))[0] == 0


# ------------------------------------------------------------------------------------------------ seeded generator
def test_generator_matches_numpy_twin():
    assert (O.synth_tokens(42, 64, 128256) == synth.prompt_tokens(64, 128256)[0]).all()
    assert (O.synth_tokens(7, 20, 1000, first=20) == synth.prompt_tokens(20, 1000, batch=2, seed=7)[1]).all()
    w = O.synth_normal_f16(synth.name_seed("layers.0.attention.wq.weight"), 1 << 18, 0.02).astype(np.float64)
    assert abs(w.mean()) < 2e-4 and abs(w.std() - 0.02) < 2e-4
    assert (O.synth_normal_f16(5, 100, 0.02, first=50) == O.synth_normal_f16(5, 150, 0.02)[50:]).all()
    q = O.synth_uniform_i8(9, 1 << 16)
    assert q.min() == -127 and q.max() == 127
    s = O.synth_scale_f16(9, 4096, synth.INT8_SCALE_BASE).astype(np.float64)
    assert s.min() >= 0.49 * synth.INT8_SCALE_BASE and s.max() <= 1.51 * synth.INT8_SCALE_BASE


# ------------------------------------------------------------------------------------------------ float64 twin
def _np_forward(p, w, tokens, eps):
    """Independent float64 Llama forward over a full sequence (no cache, causal mask), logits of the last position."""
    d, H, G = p["dim"], p["n_heads"], p["n_kv_heads"]
    hd, S = d // H, len(tokens)
    x = w["emb"][tokens]
    i = np.arange(hd // 2)
    ang = np.outer(np.arange(S), 1.0 / p["rope_theta"] ** (2 * i / hd))
    co, si = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]

    def norm(v):
        return v / np.sqrt((v * v).mean(-1, keepdims=True) + eps)

    def rope(t):
        a, b = t[..., 0::2], t[..., 1::2]
        out = np.empty_like(t)
        out[..., 0::2], out[..., 1::2] = a * co - b * si, a * si + b * co
        return out

    for l in range(p["n_layers"]):
        xn = norm(x)
        q = rope((xn @ w[l, "wq"].T).reshape(S, H, hd))
        k = rope((xn @ w[l, "wk"].T).reshape(S, G, hd))
        v = (xn @ w[l, "wv"].T).reshape(S, G, hd)
        k, v = np.repeat(k, H // G, axis=1), np.repeat(v, H // G, axis=1)
        s = np.einsum("shd,thd->hst", q, k) / math.sqrt(hd) + np.triu(np.full((S, S), -np.inf), 1)[None]
        pr = np.exp(s - s.max(-1, keepdims=True)); pr /= pr.sum(-1, keepdims=True)
        x = x + np.einsum("hst,thd->shd", pr, v).reshape(S, d) @ w[l, "wo"].T
        xn = norm(x)
        g = xn @ w[l, "w1"].T
        x = x + (g / (1 + np.exp(-g)) * (xn @ w[l, "w3"].T)) @ w[l, "w2"].T
    return norm(x[-1]) @ w["out"].T


@pytest.mark.parametrize("int8", [False, True])
def test_model_agrees_with_float64_twin(int8):
    p = TINY
    m = build_oracle(p, max_context=32, max_batch=1, int8=int8, tied=True)
    shapes = tensor_shapes(p)
    w = {}

    def deq(name, shape):
        a, s = synth_weight(name, shape, int8)
        return a.astype(np.float64) if s is None else (a.astype(np.float16) * s[:, None]).astype(np.float64)

    for l in range(p["n_layers"]):
        for short, suffix in (("wq", "attention.wq"), ("wk", "attention.wk"), ("wv", "attention.wv"), ("wo", "attention.wo"),
                              ("w1", "feed_forward.w1"), ("w2", "feed_forward.w2"), ("w3", "feed_forward.w3")):
            w[l, short] = deq(f"layers.{l}.{suffix}", shapes[suffix])
    w["emb"] = w["out"] = deq("tok_embeddings", (p["vocab_size"], p["dim"]))
    toks = synth.prompt_tokens(10, p["vocab_size"])[0]
    logits = None
    for i, t in enumerate(toks):
        logits, _ = m.forward(np.array([[t]], np.int32), i)
    ref = _np_forward(p, w, toks, p["norm_eps"])
    assert np.abs(logits[0] - ref).max() < 1e-2, np.abs(logits[0] - ref).max()
    # batched multi-token call (mask path) equals token-at-a-time
    m2 = build_oracle(p, max_context=32, max_batch=1, int8=int8, tied=True)
    logits2, _ = m2.forward(toks[None, :], 0)
    assert (logits2 == logits).all()


# ------------------------------------------------------------------------------------------------ fixtures
@pytest.mark.parametrize("name,int8", [("tiny_fp16", False), ("tiny_int8", True)])
def test_golden_tiny(name, int8):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    m = build_oracle(TINY, max_context=64, max_batch=2, int8=int8, tied=True)
    ids, logits, margins = oracle_greedy(m, g["prompt"], g["ids"].shape[1])
    assert (ids == g["ids"]).all()
    assert (logits.astype(np.float16) == g["logits"]).all()


def test_golden_c1_is_present_and_consistent():
    g = np.load(os.path.join(GOLD, "c1_llama32_1b.npz"))
    assert g["ids"].shape == (1, 64) and g["prompt"].shape == (1, 32)
    assert (g["prompt"] == synth.prompt_tokens(32, 128256, seed=int(g["prompt_seed"]))).all()
    assert (g["margins"] > 0).all()
