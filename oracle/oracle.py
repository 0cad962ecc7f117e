"""ctypes front-end of the CPU checker (``llama_oracle.c`` + ``synth.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the CPU-baseline / reference legs of
the benchmark; the shipped package never imports it.  Parity is unpinned (see the header of ``llama_oracle.c``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")

# per-layer / global tensor ids (mirror the enums in llama_oracle.c)
WQ, WK, WV, WO, W1, W2, W3, ATTN_NORM, FFN_NORM = range(9)
TOK_EMB, OUTPUT, NORM = range(3)


def build(force: bool = False) -> str:
    """Compile the checker with the committed Makefile; returns the library path."""
    srcs = [os.path.join(_HERE, f) for f in ("llama_oracle.c", "sample_oracle.c", "synth.c", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True, capture_output=True)
    return _LIB_PATH


class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dim", "n_layers", "n_heads", "n_kv_heads", "hidden", "vocab",
                                          "max_context", "max_batch", "quant", "quant_embed")] + \
               [("eps", C.c_float), ("theta", C.c_double)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        vp, i32, u64, f32, f64 = C.c_void_p, C.c_int32, C.c_uint64, C.c_float, C.c_double
        sigs = {
            "orc_xexp2_f32": (f32, [f32]), "orc_xexp2_f16": (C.c_uint16, [C.c_uint16]), "orc_xsin_f32": (f32, [f32]),
            "orc_freqs_cis": (None, [i32, i32, f64, vp]),
            "orc_rmsnorm": (None, [vp, vp, vp, i32, i32, f32]),
            "orc_linear_f16": (None, [vp, vp, vp, i32, i32, i32]),
            "orc_linear_w8": (None, [vp, vp, vp, vp, i32, i32, i32]),
            "orc_quantize_w8": (None, [vp, vp, vp, i32, i32]),
            "orc_nf4_dequant": (None, [vp, vp, vp, C.c_int64, i32]),
            "orc_nf4_quantize": (None, [vp, vp, vp, C.c_int64, i32]),
            "orc_embed_f16": (None, [vp, vp, vp, i32, i32]),
            "orc_embed_w8": (None, [vp, vp, vp, vp, i32, i32]),
            "orc_rope": (None, [vp, vp, vp, i32, i32, i32]),
            "orc_attention": (None, [vp, vp, vp, vp] + [i32] * 7),
            "orc_swiglu": (None, [vp, vp, vp, i32]),
            "orc_argmax_f16": (i32, [vp, i32]),
            "orc_model_create": (vp, [C.POINTER(_Config)]),
            "orc_model_destroy": (None, [vp]),
            "orc_model_set_weight": (None, [vp, i32, i32, vp, vp]),
            "orc_model_table": (vp, [vp]),
            "orc_model_cache": (vp, [vp]),
            "orc_set_threads": (None, [i32]), "orc_max_threads": (i32, []),
            "orc_sample": (i32, [vp, i32, f32, i32, f32, f32, f32, vp, f32]),
            "orc_sum_f32": (f32, [vp, i32]),
            "orc_threefry2x32": (u64, [u64, u64]),
            "orc_threefry_rand_f32": (None, [C.c_uint32, C.c_uint32, C.c_uint32, u64, vp]),
            "orc_model_forward": (i32, [vp, vp, i32, i32, i32, vp, vp, vp]),
            "orc_synth_normal_f16": (None, [u64, u64, u64, f32, vp]),
            "orc_synth_uniform_i8": (None, [u64, u64, u64, vp]),
            "orc_synth_scale_f16": (None, [u64, u64, u64, f32, vp]),
            "orc_synth_const_f16": (None, [u64, f32, vp]),
            "orc_synth_tokens": (None, [u64, u64, u64, i32, vp]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def set_threads(n: int) -> int:
    """Thread count of the checker's OpenMP loops from now on; returns the count in force."""
    lib().orc_set_threads(int(n))
    return int(lib().orc_max_threads())


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _h(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


# ---------------------------------------------------------------- unit ops (numpy in, numpy out)
def xexp2_f32(x: float) -> float:
    return float(lib().orc_xexp2_f32(np.float32(x)))


def xexp2_f16(x) -> np.float16:
    bits = int(np.array(x, dtype=np.float16).view(np.uint16))
    return np.array(lib().orc_xexp2_f16(bits), dtype=np.uint16).view(np.float16)[()]


def xsin_f32(x: float) -> float:
    return float(lib().orc_xsin_f32(np.float32(x)))


def freqs_cis(head_dim: int, end: int, theta: float) -> np.ndarray:
    out = np.empty((end, head_dim // 2, 2), np.float16)
    lib().orc_freqs_cis(head_dim, end, theta, _p(out))
    return out


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x, w = _h(x), _h(w)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(y), x.size // x.shape[-1], x.shape[-1], eps)
    return y


def linear_f16(x, w) -> np.ndarray:
    x, w = _h(x), _h(w)
    M, K = x.size // x.shape[-1], x.shape[-1]
    N = w.shape[0]
    assert w.shape[1] == K
    y = np.empty(x.shape[:-1] + (N,), np.float16)
    lib().orc_linear_f16(_p(x), _p(w), _p(y), M, N, K)
    return y


def linear_w8(x, wq, scale) -> np.ndarray:
    x, scale = _h(x), _h(scale)
    wq = np.ascontiguousarray(wq)
    assert wq.dtype == np.int8
    M, K = x.size // x.shape[-1], x.shape[-1]
    N = wq.shape[0]
    y = np.empty(x.shape[:-1] + (N,), np.float16)
    lib().orc_linear_w8(_p(x), _p(wq), _p(scale), _p(y), M, N, K)
    return y


def quantize_w8(w):
    w = _h(w)
    N, K = w.shape
    wq = np.empty((N, K), np.int8)
    s = np.empty((N,), np.float16)
    lib().orc_quantize_w8(_p(w), _p(wq), _p(s), N, K)
    return wq, s


def nf4_quantize(w, block: int = 64):
    """NF4Linear.quantize on one fp16 matrix: (packed uint8 [n/2], scale fp16 [n/block, 1])."""
    w = _h(w)
    n = w.size
    packed = np.empty((n // 2,), np.uint8)
    scale = np.empty((n // block, 1), np.float16)
    lib().orc_nf4_quantize(_p(w), _p(packed), _p(scale), n, block)
    return packed, scale


def nf4_dequant(packed, scale, shape, block: int = 64) -> np.ndarray:
    """The fp16 matrix NF4Linear.call multiplies by: half(CODE[code] * scale), reshaped to [out, in]."""
    packed, scale = np.ascontiguousarray(packed, dtype=np.uint8), _h(scale)
    out = np.empty((packed.size * 2,), np.float16)
    lib().orc_nf4_dequant(_p(packed), _p(scale), _p(out), out.size, block)
    return out.reshape(shape)


def embed_f16(idx, w) -> np.ndarray:
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    w = _h(w)
    out = np.empty(idx.shape + (w.shape[1],), np.float16)
    lib().orc_embed_f16(_p(idx), _p(w), _p(out), idx.size, w.shape[1])
    return out


def embed_w8(idx, wq, scale) -> np.ndarray:
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    wq = np.ascontiguousarray(wq)
    out = np.empty(idx.shape + (wq.shape[1],), np.float16)
    lib().orc_embed_w8(_p(idx), _p(wq), _p(_h(scale)), _p(out), idx.size, wq.shape[1])
    return out


def rope(x, table, pos) -> np.ndarray:
    """x [rows, n_heads, hd] (copied), table [end, hd/2, 2], pos [rows] -> rotated copy."""
    x = _h(x).copy()
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    rows, nh, hd = x.shape
    lib().orc_rope(_p(x), _p(_h(table)), _p(pos), rows, nh, hd)
    return x


def attention(q, k, v, start_pos: int) -> np.ndarray:
    """q [B,S,H,hd]; k, v [B,Tmax,G,hd] contiguous cache -> [B,S,H*hd]."""
    q, k, v = _h(q), _h(k), _h(v)
    B, S, H, hd = q.shape
    Tmax, G = k.shape[1], k.shape[2]
    out = np.empty((B, S, H * hd), np.float16)
    lib().orc_attention(_p(q), _p(k), _p(v), _p(out), B, S, H, G, hd, Tmax, start_pos)
    return out


def swiglu(g, u) -> np.ndarray:
    g, u = _h(g), _h(u)
    out = np.empty_like(g)
    lib().orc_swiglu(_p(g), _p(u), _p(out), g.size)
    return out


def argmax_f16(x) -> int:
    x = _h(x)
    return int(lib().orc_argmax_f16(_p(x), x.size))


def sample(logits, temp: float, k: int, p: float, af: float, ap: float, u: float, alpha_counter: np.ndarray | None = None) -> int:
    """`sample` of jsgrad/models/llama.ts:131-185 on one row of float32 logits with the uniform sample `u`;
    `alpha_counter` (int32 [n]) is updated in place when a penalty is active."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    if alpha_counter is not None:
        assert alpha_counter.dtype == np.int32 and alpha_counter.flags["C_CONTIGUOUS"] and alpha_counter.size == logits.size
    return int(lib().orc_sample(_p(logits), logits.size, temp, k, p, af, ap, _p(alpha_counter), u))


def sum_f32(x) -> float:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return float(lib().orc_sum_f32(_p(x), x.size))


def threefry_rand(seed0: int, seed1: int, counter: int, num: int) -> np.ndarray:
    """float32 [num] in [0, 1): the values one Tensor.rand call of `num` float32 elements produces
    (jsgrad/tensor.ts:796-843) for the seed pair (device hash, Tensor._seed) and the device's counter."""
    out = np.empty((num,), np.float32)
    lib().orc_threefry_rand_f32(seed0 & 0xFFFFFFFF, seed1 & 0xFFFFFFFF, counter & 0xFFFFFFFF, num, _p(out))
    return out


# ---------------------------------------------------------------- seeded generator
def synth_normal_f16(seed: int, n: int, std: float, first: int = 0) -> np.ndarray:
    out = np.empty(n, np.float16)
    lib().orc_synth_normal_f16(seed, first, n, std, _p(out))
    return out


def synth_uniform_i8(seed: int, n: int, first: int = 0) -> np.ndarray:
    out = np.empty(n, np.int8)
    lib().orc_synth_uniform_i8(seed, first, n, _p(out))
    return out


def synth_scale_f16(seed: int, n: int, base: float, first: int = 0) -> np.ndarray:
    out = np.empty(n, np.float16)
    lib().orc_synth_scale_f16(seed, first, n, base, _p(out))
    return out


def synth_tokens(seed: int, n: int, vocab: int, first: int = 0) -> np.ndarray:
    out = np.empty(n, np.int32)
    lib().orc_synth_tokens(seed, first, n, vocab, _p(out))
    return out


# ---------------------------------------------------------------- whole model
@dataclass
class OracleConfig:
    dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    hidden: int
    vocab: int
    max_context: int
    max_batch: int = 1
    quant: int = 0
    quant_embed: int = 0
    eps: float = 1e-5
    theta: float = 500000.0


class OracleModel:
    """Holds borrowed numpy weights and the KV cache; ``forward`` follows Transformer.forward."""

    def __init__(self, cfg: OracleConfig):
        self.cfg = cfg
        c = _Config(cfg.dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.hidden, cfg.vocab, cfg.max_context,
                    cfg.max_batch, cfg.quant, cfg.quant_embed, cfg.eps, cfg.theta)
        self._m = lib().orc_model_create(C.byref(c))
        self._keep: list[np.ndarray] = []

    def set_weight(self, layer: int, which: int, w: np.ndarray, scale: np.ndarray | None = None):
        w = np.ascontiguousarray(w)
        self._keep.append(w)
        if scale is not None:
            scale = np.ascontiguousarray(scale)
            self._keep.append(scale)
        lib().orc_model_set_weight(self._m, layer, which, _p(w), _p(scale))

    def table(self) -> np.ndarray:
        hd = self.cfg.dim // self.cfg.n_heads
        n = 2 * self.cfg.max_context * hd
        buf = (C.c_uint16 * n).from_address(lib().orc_model_table(self._m))
        return np.frombuffer(buf, dtype=np.float16).reshape(2 * self.cfg.max_context, hd // 2, 2)

    def cache(self) -> np.ndarray:
        """The KV cache as a writable fp16 view [L][2][B][max_context][G][hd] (timing runs fill it with stand-in rows
        instead of computing a long prompt)."""
        c = self.cfg
        hd = c.dim // c.n_heads
        shape = (c.n_layers, 2, c.max_batch, c.max_context, c.n_kv_heads, hd)
        buf = (C.c_uint16 * int(np.prod(shape))).from_address(lib().orc_model_cache(self._m))
        return np.frombuffer(buf, dtype=np.float16).reshape(shape)

    def forward(self, tokens, start_pos: int, want_hidden: bool = False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        B, S = tokens.shape
        logits = np.empty((B, self.cfg.vocab), np.float32)
        nxt = np.empty((B,), np.int32)
        hidden = np.empty((B, S, self.cfg.dim), np.float16) if want_hidden else None
        rc = lib().orc_model_forward(self._m, _p(tokens), B, S, start_pos, _p(logits), _p(nxt), _p(hidden))
        if rc != 0:
            raise ValueError("oracle forward: batch or context exceeds the configured maximum")
        return (logits, nxt, hidden) if want_hidden else (logits, nxt)

    def close(self):
        if self._m:
            lib().orc_model_destroy(self._m)
            self._m = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
