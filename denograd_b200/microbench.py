"""Per-kernel timings through the C ABI, for choosing the library's environment knobs on a given machine
(`JG_TC_SPLITK`, `JG_TC_PAIR`, `JG_ATTN_CLUSTER`, `JG_ATTN_STAGES`, ...: they are read once per process, so run one
process per setting) and for checking a kernel in isolation:

    python -m denograd_b200.microbench projections --rows 512          # the four projections of a layer
    python -m denograd_b200.microbench prefill-attention --positions 512 --start 0
    python -m denograd_b200.microbench decode-attention --batch 32 --context 4100

Shapes default to the Llama-3.1-8B architecture (`--dim --hidden --heads --kv-heads`).  Every launch is timed alone with
CUDA events on the device's stream (`jg_timer_start` / `jg_timer_stop`) after 256 MB of memset have displaced the L2
contents, so the figures are cold-cache ones: inside a model's step the same launches overlap their neighbours and find
their activations in L2.  The median of `--repeat` launches is printed.
"""
from __future__ import annotations

import argparse

import numpy as np

from . import Device
from .device import Tensor
from .llama import KVCache, precompute_freqs_cis


def _time(dev, flush: Tensor, fn, repeat: int) -> float:
    fn()
    dev.synchronize()
    ts = []
    for i in range(repeat):
        dev.call("jg_memset", flush.ptr, i & 0xFF, flush.nbytes)
        dev.timer_start()
        fn()
        ts.append(dev.timer_stop() * 1e6)
    return float(np.median(ts))


def projections(a) -> None:
    dev = Device["CUDA"]
    rng = np.random.default_rng(0)
    M, dim, hid = a.rows, a.dim, a.hidden
    hd = dim // a.heads
    qkv_n = (a.heads + 2 * a.kv_heads) * hd

    def T(shape, s=0.05):
        return Tensor((rng.standard_normal(shape) * s).astype(np.float16), device=dev)

    x, xh, res = T((M, dim), 0.5), T((M, hid), 0.5), T((M, dim), 0.5)
    wqkv, wo, w1, w3, w2 = T((qkv_n, dim)), T((dim, dim)), T((hid, dim)), T((hid, dim)), T((dim, hid))
    yq, yo, yf = Tensor.empty((M, qkv_n), "float16", dev), Tensor.empty((M, dim), "float16", dev), Tensor.empty((M, hid), "float16", dev)
    flush = Tensor.zeros((256 << 20,), "uint8", dev)
    cases = [
        ("qkv", 2 * M * qkv_n * dim, (qkv_n * dim) * 2, lambda: dev.call("jg_linear", yq.ptr, x.ptr, wqkv.ptr, 0, 0, M, qkv_n, dim)),
        ("wo + residual", 2 * M * dim * dim, dim * dim * 2, lambda: dev.call("jg_linear", yo.ptr, x.ptr, wo.ptr, 0, res.ptr, M, dim, dim)),
        ("gate/up + SwiGLU", 4 * M * hid * dim, 2 * hid * dim * 2,
         lambda: dev.call("jg_norm_swiglu", yf.ptr, x.ptr, 0, 1e-5, w1.ptr, 0, w3.ptr, 0, M, hid, dim)),
        ("down + residual", 2 * M * dim * hid, dim * hid * 2, lambda: dev.call("jg_linear", yo.ptr, xh.ptr, w2.ptr, 0, res.ptr, M, dim, hid)),
    ]
    total, flops = 0.0, 0
    for name, fl, wbytes, fn in cases:
        t = _time(dev, flush, fn, a.repeat)
        total += t
        flops += fl
        print(f"rows {M:5d}  {name:18s} {t:8.1f} us  {fl / t / 1e6:7.0f} TFLOP/s  {wbytes / t / 1e3:7.0f} GB/s of weights")
    print(f"rows {M:5d}  {'layer':18s} {total:8.1f} us  {flops / total / 1e6:7.0f} TFLOP/s")


def prefill_attention(a) -> None:
    dev = Device["CUDA"]
    rng = np.random.default_rng(0)
    H, G, hd, B, Sc, start = a.heads, a.kv_heads, a.dim // a.heads, a.batch, a.positions, a.start
    max_ctx = ((start + Sc + 63) // 64) * 64
    kv = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=64)
    freqs = precompute_freqs_cis(hd, 2 * max_ctx, 500000.0, dev)
    stride = (H + 2 * G) * hd

    def rows(t0, n):
        q = Tensor((rng.standard_normal((n * B, stride)) * 0.7).astype(np.float16), device=dev)
        p = Tensor(np.repeat(np.arange(t0, t0 + n, dtype=np.int32), B), device=dev)
        s = Tensor(np.tile(np.arange(B, dtype=np.int32), n), device=dev)
        dev.call("jg_rope_kvwrite_rows", kv.handle, 0, q.ptr, freqs.ptr, freqs.shape[0], p.ptr, s.ptr, n * B, H)
        return q, p, s

    if start:
        rows(0, start)
    q, p, s = rows(start, Sc)
    out = Tensor.zeros((Sc * B, H * hd), "float16", dev)
    flush = Tensor.zeros((256 << 20,), "uint8", dev)
    t = _time(dev, flush, lambda: dev.call("jg_attn_chunk", kv.handle, 0, out.ptr, q.ptr, p.ptr, s.ptr, B, Sc, H), a.repeat)
    pairs = B * H * (Sc * start + Sc * (Sc + 1) // 2)  # (query, key) pairs under the causal mask
    print(f"prefill attention  {Sc} positions after {start}, batch {B}: {t:8.1f} us  {4 * pairs * hd / t / 1e6:6.0f} TFLOP/s (q.k and p.v once each)")
    kv.close()


def decode_attention(a) -> None:
    dev = Device["CUDA"]
    rng = np.random.default_rng(0)
    H, G, hd, B, ctx = a.heads, a.kv_heads, a.dim // a.heads, a.batch, a.context
    max_ctx = ((ctx + 63) // 64 + 1) * 64
    kv = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=64)
    freqs = precompute_freqs_cis(hd, 2 * max_ctx, 500000.0, dev)
    qkv = Tensor((rng.standard_normal((B, (H + 2 * G) * hd)) * 0.5).astype(np.float16), device=dev)
    pos = Tensor(np.full((B,), ctx - 1, np.int32), device=dev)
    out = Tensor.empty((B, H * hd), "float16", dev)
    flush = Tensor.zeros((256 << 20,), "uint8", dev)
    t = _time(dev, flush, lambda: dev.call("jg_attn_decode_fused", kv.handle, 0, out.ptr, qkv.ptr, freqs.ptr, freqs.shape[0], pos.ptr, B, H), a.repeat)
    kv_bytes = 2 * B * ctx * G * hd * 2
    print(f"decode attention   batch {B} over {ctx} positions (unwritten cache rows read as stored: zeros): {t:8.1f} us  {kv_bytes / t / 1e3:6.0f} GB/s of K and V")
    kv.close()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["projections", "prefill-attention", "decode-attention"])
    ap.add_argument("--rows", type=int, default=512, help="activation rows of the projections")
    ap.add_argument("--positions", type=int, default=512, help="new positions of the prefill chunk")
    ap.add_argument("--start", type=int, default=0, help="positions already in the cache before the chunk")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=4100, help="context length of the decode step")
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=14336)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--repeat", type=int, default=10)
    a = ap.parse_args(argv)
    {"projections": projections, "prefill-attention": prefill_attention, "decode-attention": decode_attention}[a.what](a)


if __name__ == "__main__":
    main()
