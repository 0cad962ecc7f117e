"""GPU parity of each kernel against the CPU checker, through the C ABI (via the package's ctypes binding).

Bars: integer / index / elementwise-fp16 work is bit-exact (the device restates the reference's op-by-op fp16 and
polynomial arithmetic); reductions accumulate in fp32 in a different order than the checker's sequential loop, so
their fp16 outputs may differ by at most one fp16 unit in the last place, on a small fraction of the elements.
"""
import ctypes as C

import numpy as np
import pytest

from denograd_b200 import ffi, synth
from denograd_b200.device import Tensor
from denograd_b200.llama import KVCache, precompute_freqs_cis
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def ulp_diff(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in fp16 units in the last place (monotonic integer mapping of the bit patterns)."""
    def key(x):
        u = np.ascontiguousarray(x, dtype=np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    return np.abs(key(a) - key(b))


def assert_reduction_close(got, ref, max_ulp=1, max_frac=0.03, what=""):
    assert got.shape == ref.shape
    assert np.isfinite(got.astype(np.float32)).all(), what
    d = ulp_diff(got, ref)
    # near zero an "ulp" is tiny; there fall back to an absolute bound of one ulp of the row scale
    scale = np.maximum(np.abs(ref.astype(np.float32)).max(), 1e-6)
    bad = (d > max_ulp) & (np.abs(got.astype(np.float32) - ref.astype(np.float32)) > scale * 2.0 ** -10)
    assert not bad.any(), f"{what}: {bad.sum()} elements differ by more than {max_ulp} ulp (max {d.max()})"
    assert (d > 0).mean() <= max_frac, f"{what}: {(d > 0).mean():.4f} of the elements differ"


# ------------------------------------------------------------------------------------------------ bit-exact kernels
def test_seeded_fills_match_cpu_generator(dev):
    n = 100_003
    t = Tensor.empty((n,), "float16", dev)
    dev.call("jg_fill_normal_f16", t.ptr, 77, 5, n, 0.02)
    assert (t.numpy().view(np.uint16) == O.synth_normal_f16(77, n, 0.02, first=5).view(np.uint16)).all()
    q = Tensor.empty((n,), "int8", dev)
    dev.call("jg_fill_uniform_i8", q.ptr, 78, 0, n)
    assert (q.numpy() == O.synth_uniform_i8(78, n)).all()
    s = Tensor.empty((n,), "float16", dev)
    dev.call("jg_fill_scale_f16", s.ptr, 79, 11, n, synth.INT8_SCALE_BASE)
    assert (s.numpy().view(np.uint16) == O.synth_scale_f16(79, n, synth.INT8_SCALE_BASE, first=11).view(np.uint16)).all()
    dev.call("jg_fill_const_f16", s.ptr, n, 1.0)
    assert (s.numpy() == 1.0).all()


@pytest.mark.parametrize("hd,end", [(64, 512), (128, 16384)])
def test_freqs_cis_bit_exact(dev, hd, end):
    got = precompute_freqs_cis(hd, end, 500000.0, dev).numpy()
    ref = O.freqs_cis(hd, end, 500000.0)
    assert (got.view(np.uint16) == ref.view(np.uint16)).all()


def test_embedding_gather(dev):
    rng = np.random.default_rng(0)
    V, d = 777, 256
    w = rng.standard_normal((V, d)).astype(np.float16)
    idx = np.array([[0, 776, 5], [5, 13, 400]], np.int32)
    out = Tensor.empty((2, 3, d), "float16", dev)
    # device tensors are bound to names: a temporary's buffer returns to the allocator's cache as soon as the
    # expression ends and the next upload of the same size would overwrite it
    it, wt = Tensor(idx, device=dev), Tensor(w, device=dev)
    dev.call("jg_embed", out.ptr, it.ptr, wt.ptr, 0, idx.size, d, V)
    assert (out.numpy() == O.embed_f16(idx, w)).all()
    wq = rng.integers(-127, 128, (V, d), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, V) * 3e-4).astype(np.float16)
    qt, st = Tensor(wq, device=dev), Tensor(s, device=dev)
    dev.call("jg_embed", out.ptr, it.ptr, qt.ptr, st.ptr, idx.size, d, V)
    assert (out.numpy().view(np.uint16) == O.embed_w8(idx, wq, s).view(np.uint16)).all()
    # an index outside the table selects no row: zeros, as the reference's one-hot sum gives
    bad = np.array([V, -1], np.int32)
    out2 = Tensor.empty((2, d), "float16", dev)
    bt = Tensor(bad, device=dev)
    dev.call("jg_embed", out2.ptr, bt.ptr, wt.ptr, 0, 2, d, V)
    assert (out2.numpy() == 0).all()


def test_swiglu_elementwise_bit_exact(dev):
    g = np.concatenate([np.linspace(-40, 40, 8000), [0.0, -0.0, 65504, -65504, 1e-7, 23, -23, 22.5]]).astype(np.float16)
    u = np.resize(np.linspace(-3, 3, 97).astype(np.float16), g.shape)
    y = Tensor.empty(g.shape, "float16", dev)
    gt, ut = Tensor(g, device=dev), Tensor(u, device=dev)
    dev.call("jg_swiglu", y.ptr, gt.ptr, ut.ptr, g.size)
    assert (y.numpy().view(np.uint16) == O.swiglu(g, u).view(np.uint16)).all()


def test_argmax_lowest_index(dev):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 128256)).astype(np.float16)
    x[0, [70000, 90000]] = 9.0
    x[1, :] = -1.0
    x[2, 128255] = 11.0
    out = Tensor.empty((3,), "int32", dev)
    xt = Tensor(x, device=dev)
    dev.call("jg_argmax", out.ptr, xt.ptr, 3, x.shape[1])
    assert out.numpy().tolist() == [70000, 0, 128255]
    assert out.numpy().tolist() == [O.argmax_f16(r) for r in x]


# ------------------------------------------------------------------------------------------------ reductions
def test_rmsnorm(dev):
    rng = np.random.default_rng(2)
    for rows, d in [(1, 2048), (5, 3072), (2, 8192)]:
        x = (rng.standard_normal((rows, d)) * 1.7).astype(np.float16)
        w = rng.uniform(0.5, 1.5, d).astype(np.float16)
        y = Tensor.empty((rows, d), "float16", dev)
        xt, wt = Tensor(x, device=dev), Tensor(w, device=dev)
        dev.call("jg_rmsnorm", y.ptr, xt.ptr, wt.ptr, rows, d, 1e-5)
        assert_reduction_close(y.numpy(), O.rmsnorm(x, w, 1e-5), what=f"rmsnorm {rows}x{d}")


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 8])
@pytest.mark.parametrize("int8", [False, True])
def test_linear(dev, M, int8):
    rng = np.random.default_rng(10 * M + int8)
    for N, K in [(64, 256), (1027, 2048), (333, 1040), (2048, 8192)]:  # odd row counts and ragged K chunks
        if int8 and K % 16:
            continue
        x = rng.standard_normal((M, K)).astype(np.float16)
        res = rng.standard_normal((M, N)).astype(np.float16)
        y = Tensor.empty((M, N), "float16", dev)
        xt = Tensor(x, device=dev)
        if int8:
            wq = rng.integers(-127, 128, (N, K), dtype=np.int8)
            s = (rng.uniform(0.5, 1.5, N) * synth.INT8_SCALE_BASE).astype(np.float16)
            wt, st = Tensor(wq, device=dev), Tensor(s, device=dev)
            ref = O.linear_w8(x, wq, s)
            sp = st.ptr
        else:
            w = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
            wt, sp = Tensor(w, device=dev), 0
            ref = O.linear_f16(x, w)
        dev.call("jg_linear", y.ptr, xt.ptr, wt.ptr, sp, 0, M, N, K)
        assert_reduction_close(y.numpy(), ref, what=f"linear M{M} N{N} K{K} int8={int8}")
        # residual epilogue: fp16 add of the rounded projection
        rt = Tensor(res, device=dev)
        dev.call("jg_linear", y.ptr, xt.ptr, wt.ptr, sp, rt.ptr, M, N, K)
        ref_r = (res.astype(np.float32) + ref.astype(np.float32)).astype(np.float16)  # exact sum, one rounding
        assert_reduction_close(y.numpy(), ref_r, max_ulp=2, max_frac=0.05, what=f"linear+residual M{M} N{N} K{K}")


@pytest.mark.parametrize("M,int8", [(1, False), (4, False), (1, True), (2, True)])
def test_fused_norm_projections(dev, M, int8):
    rng = np.random.default_rng(100 + M)
    K, N, F = 2048, 1536, 1024
    x = (rng.standard_normal((M, K)) * 0.8).astype(np.float16)
    g = rng.uniform(0.5, 1.5, K).astype(np.float16)
    xn = O.rmsnorm(x, g, 1e-5)

    def mk(n):
        if int8:
            wq = rng.integers(-127, 128, (n, K), dtype=np.int8)
            s = (rng.uniform(0.5, 1.5, n) * synth.INT8_SCALE_BASE).astype(np.float16)
            return (wq, s), (Tensor(wq, device=dev), Tensor(s, device=dev))
        w = (rng.standard_normal((n, K)) * 0.02).astype(np.float16)
        return (w, None), (Tensor(w, device=dev), None)

    def lin(h, a):
        return O.linear_w8(a, *h) if int8 else O.linear_f16(a, h[0])

    xt, gt = Tensor(x, device=dev), Tensor(g, device=dev)
    h, (wt, st) = mk(N)
    y = Tensor.empty((M, N), "float16", dev)
    dev.call("jg_norm_linear", y.ptr, xt.ptr, gt.ptr, 1e-5, wt.ptr, st.ptr if st else 0, M, N, K)
    # the fused prologue sums x^2 in another order than the checker: the normaliser may move by one fp32 ulp, a few
    # normalised inputs then round the other way in fp16, and that nudges a larger share of the outputs by one ulp
    assert_reduction_close(y.numpy(), lin(h, xn), max_ulp=2, max_frac=0.20, what="norm_linear")

    h1, (w1, s1) = mk(F)
    h3, (w3, s3) = mk(F)
    f = Tensor.empty((M, F), "float16", dev)
    dev.call("jg_norm_swiglu", f.ptr, xt.ptr, gt.ptr, 1e-5, w1.ptr, s1.ptr if s1 else 0, w3.ptr, s3.ptr if s3 else 0, M, F, K)
    ref = O.swiglu(lin(h1, xn), lin(h3, xn))
    assert_reduction_close(f.numpy(), ref, max_ulp=3, max_frac=0.25, what="norm_swiglu")

    V = 5003
    hv, (wv, sv) = mk(V)
    logits = Tensor.empty((M, V), "float16", dev)
    key = Tensor.zeros((M,), "uint64", dev)
    tok = Tensor.empty((M,), "int32", dev)
    dev.call("jg_norm_logits_argmax", logits.ptr, key.ptr, xt.ptr, gt.ptr, 1e-5, wv.ptr, sv.ptr if sv else 0, M, V, K)
    dev.call("jg_argmax_finalize", tok.ptr, key.ptr, M)
    got = logits.numpy()
    assert_reduction_close(got, lin(hv, xn), max_ulp=2, max_frac=0.20, what="logits")
    assert tok.numpy().tolist() == [O.argmax_f16(r) for r in got]  # greedy pick is the lowest-index max of its own logits
    assert (key.numpy() == 0).all()


@pytest.mark.parametrize("M", [9, 16, 17, 32, 40, 64])
@pytest.mark.parametrize("int8", [False, True])
def test_tensor_core_projection(dev, M, int8):
    """8 < M <= 64 rows: mma.sync path (and tcgen05 where the shape allows it), fp16 and int8 weights, every epilogue,
    ragged N / K, all K-split variants (chosen from N)."""
    rng = np.random.default_rng(500 + M + int8)

    def mk(n, k):
        if int8:
            wq = rng.integers(-127, 128, (n, k), dtype=np.int8)
            sc = (rng.uniform(0.5, 1.5, n) * synth.INT8_SCALE_BASE).astype(np.float16)
            wt, st = Tensor(wq, device=dev), Tensor(sc, device=dev)
            return (wt, st), st.ptr, (lambda a: O.linear_w8(a, wq, sc))
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float16)
        wt = Tensor(w, device=dev)
        return (wt, None), 0, (lambda a: O.linear_f16(a, w))

    for N, K in [(64, 256), (1027, 2048), (333, 1040), (2048, 8192), (40000, 512)]:
        x = rng.standard_normal((M, K)).astype(np.float16)
        res = rng.standard_normal((M, N)).astype(np.float16)
        xt, rt = Tensor(x, device=dev), Tensor(res, device=dev)
        (wt, keep), sp, lin = mk(N, K)
        y = Tensor.empty((M, N), "float16", dev)
        ref = lin(x)
        dev.call("jg_linear", y.ptr, xt.ptr, wt.ptr, sp, 0, M, N, K)
        assert_reduction_close(y.numpy(), ref, max_ulp=1, max_frac=0.05, what=f"mma linear M{M} N{N} K{K} int8={int8}")
        dev.call("jg_linear", y.ptr, xt.ptr, wt.ptr, sp, rt.ptr, M, N, K)
        ref_r = (res.astype(np.float32) + ref.astype(np.float32)).astype(np.float16)
        assert_reduction_close(y.numpy(), ref_r, max_ulp=2, max_frac=0.06, what=f"mma linear+residual M{M} N{N} K{K}")
        p32 = Tensor.zeros((M, N), "float32", dev)
        dev.call("jg_linear_partial", p32.ptr, xt.ptr, wt.ptr, sp, M, N, K)
        assert np.abs(p32.numpy().astype(np.float16).astype(np.float32) - ref.astype(np.float32)).max() <= 2e-2
        if N <= 2048:
            (w3t, keep3), sp3, lin3 = mk(N, K)
            dev.call("jg_norm_swiglu", y.ptr, xt.ptr, 0, 1e-5, wt.ptr, sp, w3t.ptr, sp3, M, N, K)
            assert_reduction_close(y.numpy(), O.swiglu(ref, lin3(x)), max_ulp=3, max_frac=0.12, what=f"mma swiglu M{M} N{N} K{K}")
        key = Tensor.zeros((M,), "uint64", dev)
        tok = Tensor.empty((M,), "int32", dev)
        dev.call("jg_norm_logits_argmax", y.ptr, key.ptr, xt.ptr, 0, 1e-5, wt.ptr, sp, M, N, K)
        dev.call("jg_argmax_finalize", tok.ptr, key.ptr, M)
        got = y.numpy()
        assert_reduction_close(got, ref, max_ulp=1, max_frac=0.05, what=f"mma logits M{M} N{N} K{K}")
        assert tok.numpy().tolist() == [O.argmax_f16(r) for r in got]


# ------------------------------------------------------------------------------------------------ RoPE + attention
@pytest.mark.parametrize("hd,H,G", [(64, 32, 8), (128, 24, 8), (128, 8, 8), (64, 4, 2), (128, 16, 2)])
@pytest.mark.parametrize("B,T,n_split", [(1, 1, 0), (1, 97, 0), (2, 300, 3), (1, 1000, 0), (3, 65, 1), (6, 130, 0)])
def test_rope_cache_attention(dev, hd, H, G, B, T, n_split):
    rng = np.random.default_rng(hd + H + T)
    max_ctx = 1024
    kv = KVCache(dev, 2, H, G, hd, max_ctx, B, page_size=64, n_split=n_split)
    # scatter the pages: row b's i-th page is an arbitrary pool page
    table = rng.permutation(kv.n_pages).astype(np.int32).reshape(B, kv.max_pages_per_seq)
    kv.set_block_table(table)
    freqs = precompute_freqs_cis(hd, 2 * max_ctx, 500000.0, dev)
    ftab = freqs.numpy()
    stride = (H + 2 * G) * hd
    qkv_all = (rng.standard_normal((T, B, stride)) * 0.7).astype(np.float16)
    layer = 1
    k_ref = np.zeros((B, max_ctx, G, hd), np.float16)
    v_ref = np.zeros((B, max_ctx, G, hd), np.float16)
    qkv = Tensor.empty((B, stride), "float16", dev)
    pos = Tensor.zeros((B,), "int32", dev)
    q_rot = None
    for t in range(T):
        qkv.assign(qkv_all[t])
        pos.assign(np.full((B,), t, np.int32))
        dev.call("jg_rope_kvwrite", kv.handle, layer, qkv.ptr, freqs.ptr, freqs.shape[0], pos.ptr, B, H)
        q_in = qkv_all[t][:, :H * hd].reshape(B, H, hd)
        k_in = qkv_all[t][:, H * hd:(H + G) * hd].reshape(B, G, hd)
        k_ref[:, t] = O.rope(k_in, ftab, [t] * B)
        v_ref[:, t] = qkv_all[t][:, (H + G) * hd:].reshape(B, G, hd)
        if t == T - 1:
            q_rot = O.rope(q_in, ftab, [t] * B)
            got_q = qkv.numpy()[:, :H * hd].reshape(B, H, hd)
            assert (got_q.view(np.uint16) == q_rot.view(np.uint16)).all(), "rotated Q differs"
    out = Tensor.empty((B, H * hd), "float16", dev)
    dev.call("jg_attn_decode", kv.handle, layer, out.ptr, qkv.ptr, pos.ptr, B, H)
    ref = O.attention(q_rot.reshape(B, 1, H, hd), k_ref, v_ref, T - 1).reshape(B, H * hd)
    assert_reduction_close(out.numpy(), ref, max_ulp=2, max_frac=0.10, what=f"attention hd{hd} H{H} G{G} B{B} T{T}")
    # a second launch reuses the scratch and tickets and must reproduce the result bit for bit
    out2 = Tensor.empty((B, H * hd), "float16", dev)
    dev.call("jg_attn_decode", kv.handle, layer, out2.ptr, qkv.ptr, pos.ptr, B, H)
    assert (out2.numpy().view(np.uint16) == out.numpy().view(np.uint16)).all()
    # the one-launch cluster kernel redoes the last position from the unrotated projections: RoPE, cache write (into
    # another layer's pages, whose earlier rows are copied from this one) and attention
    kv2 = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=64)
    kv2.set_block_table(table)
    for t in range(T - 1):
        qkv.assign(qkv_all[t])
        pos.assign(np.full((B,), t, np.int32))
        dev.call("jg_rope_kvwrite", kv2.handle, 0, qkv.ptr, freqs.ptr, freqs.shape[0], pos.ptr, B, H)
    qkv.assign(qkv_all[T - 1])
    pos.assign(np.full((B,), T - 1, np.int32))
    out3 = Tensor.empty((B, H * hd), "float16", dev)
    dev.call("jg_attn_decode_fused", kv2.handle, 0, out3.ptr, qkv.ptr, freqs.ptr, freqs.shape[0], pos.ptr, B, H)
    assert_reduction_close(out3.numpy(), ref, max_ulp=2, max_frac=0.10, what=f"fused attention hd{hd} H{H} G{G} B{B} T{T}")
    assert (qkv.numpy() == qkv_all[T - 1]).all()  # the fused kernel leaves the projections untouched
    kv.close()
    kv2.close()


@pytest.mark.parametrize("page", [16, 32, 64])
@pytest.mark.parametrize("hd,H,G,B,T", [(128, 32, 8, 2, 333), (64, 16, 8, 4, 70), (128, 8, 8, 3, 1)])
def test_fused_attention_page_sizes(dev, hd, H, G, B, T, page):
    """The one-launch decode attention over pages smaller than and equal to its staged tile of 64 positions (16 or more
    (row, kv head) pairs: the tensor-core variant), pages scattered over the pool."""
    rng = np.random.default_rng(hd + H + T + page)
    max_ctx = 512
    kv = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=page)
    table = rng.permutation(kv.n_pages).astype(np.int32).reshape(B, kv.max_pages_per_seq)
    kv.set_block_table(table)
    freqs = precompute_freqs_cis(hd, 2 * max_ctx, 500000.0, dev)
    ftab = freqs.numpy()
    stride = (H + 2 * G) * hd
    qkv_all = (rng.standard_normal((T, B, stride)) * 0.7).astype(np.float16)
    k_ref = np.zeros((B, max_ctx, G, hd), np.float16)
    v_ref = np.zeros((B, max_ctx, G, hd), np.float16)
    qkv = Tensor.empty((B, stride), "float16", dev)
    pos = Tensor.zeros((B,), "int32", dev)
    for t in range(T):
        qkv.assign(qkv_all[t])
        pos.assign(np.full((B,), t, np.int32))
        if t < T - 1:
            dev.call("jg_rope_kvwrite", kv.handle, 0, qkv.ptr, freqs.ptr, freqs.shape[0], pos.ptr, B, H)
        k_ref[:, t] = O.rope(qkv_all[t][:, H * hd:(H + G) * hd].reshape(B, G, hd), ftab, [t] * B)
        v_ref[:, t] = qkv_all[t][:, (H + G) * hd:].reshape(B, G, hd)
    q_rot = O.rope(qkv_all[T - 1][:, :H * hd].reshape(B, H, hd), ftab, [T - 1] * B)
    out = Tensor.empty((B, H * hd), "float16", dev)
    dev.call("jg_attn_decode_fused", kv.handle, 0, out.ptr, qkv.ptr, freqs.ptr, freqs.shape[0], pos.ptr, B, H)
    ref = O.attention(q_rot.reshape(B, 1, H, hd), k_ref, v_ref, T - 1).reshape(B, H * hd)
    assert_reduction_close(out.numpy(), ref, max_ulp=2, max_frac=0.10, what=f"fused attention page {page} hd{hd} B{B} T{T}")
    kv.close()


@pytest.mark.parametrize("hd,H,G", [(64, 32, 8), (128, 24, 8), (128, 8, 8), (64, 4, 2), (128, 16, 2)])
@pytest.mark.parametrize("B,start,Sc", [(1, 0, 16), (1, 0, 200), (2, 37, 75), (3, 130, 9), (1, 500, 140)])
def test_chunk_attention_on_tensor_cores(dev, hd, H, G, B, start, Sc):
    """jg_rope_kvwrite_rows + jg_attn_chunk for Sc new positions after `start` cached ones, against the checker's
    masked attention and against the row-by-row kernel."""
    rng = np.random.default_rng(hd * 7 + H + start + Sc)
    max_ctx = 1024
    kv = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=64)
    table = rng.permutation(kv.n_pages).astype(np.int32).reshape(B, kv.max_pages_per_seq)
    kv.set_block_table(table)
    freqs = precompute_freqs_cis(hd, 2 * max_ctx, 500000.0, dev)
    ftab = freqs.numpy()
    stride = (H + 2 * G) * hd
    T = start + Sc
    qkv_all = (rng.standard_normal((T, B, stride)) * 0.7).astype(np.float16)  # [position][sequence]
    k_ref = np.zeros((B, max_ctx, G, hd), np.float16)
    v_ref = np.zeros((B, max_ctx, G, hd), np.float16)
    q_ref = np.zeros((B, T, H, hd), np.float16)
    for t in range(T):
        q_ref[:, t] = O.rope(qkv_all[t][:, :H * hd].reshape(B, H, hd), ftab, [t] * B)
        k_ref[:, t] = O.rope(qkv_all[t][:, H * hd:(H + G) * hd].reshape(B, G, hd), ftab, [t] * B)
        v_ref[:, t] = qkv_all[t][:, (H + G) * hd:].reshape(B, G, hd)
    seq_of = np.tile(np.arange(B, dtype=np.int32), T)

    def rows(t0, n):
        q = Tensor(np.ascontiguousarray(qkv_all[t0:t0 + n].reshape(n * B, stride)), device=dev)
        p = Tensor(np.repeat(np.arange(t0, t0 + n, dtype=np.int32), B), device=dev)
        s = Tensor(seq_of[:n * B].copy(), device=dev)
        dev.call("jg_rope_kvwrite_rows", kv.handle, 0, q.ptr, freqs.ptr, freqs.shape[0], p.ptr, s.ptr, n * B, H)
        return q, p, s

    if start:
        keep = rows(0, start)  # the cached prefix
    q, p, s = rows(start, Sc)
    out = Tensor.zeros((Sc * B, H * hd), "float16", dev)
    dev.call("jg_attn_chunk", kv.handle, 0, out.ptr, q.ptr, p.ptr, s.ptr, B, Sc, H)
    got = out.numpy().reshape(Sc, B, H * hd).transpose(1, 0, 2)
    ref = O.attention(q_ref[:, start:], k_ref, v_ref, start)
    assert_reduction_close(got, ref, max_ulp=2, max_frac=0.12, what=f"chunk attention hd{hd} H{H} G{G} B{B} {start}+{Sc}")
    out2 = Tensor.zeros((Sc * B, H * hd), "float16", dev)
    dev.call("jg_attn_rows", kv.handle, 0, out2.ptr, q.ptr, p.ptr, s.ptr, Sc * B, H)
    assert_reduction_close(out.numpy(), out2.numpy(), max_ulp=2, max_frac=0.12, what="chunk vs row-by-row attention")
    dev.synchronize()
    kv.close()


# ------------------------------------------------------------------------------------------------ error behaviour
def test_invalid_arguments_are_rejected_before_launch(dev):
    x = Tensor.zeros((8, 64), "float16", dev)
    w = Tensor.zeros((16, 64), "float16", dev)
    y = Tensor.zeros((8, 16), "float16", dev)
    with pytest.raises(ffi.JgError) as e:
        dev.call("jg_linear", y.ptr, x.ptr, w.ptr + 2, 0, 0, 1, 16, 64)  # misaligned weight pointer
    assert e.value.status == ffi.JG_EINVAL
    with pytest.raises(ffi.JgError) as e:
        dev.call("jg_linear", y.ptr, x.ptr, w.ptr, 0, 0, 1, 16, 60)  # K not a multiple of 8
    assert e.value.status == ffi.JG_EINVAL
    with pytest.raises(ffi.JgError) as e:
        dev.call("jg_linear", y.ptr, 0, w.ptr, 0, 0, 1, 16, 64)  # null activation pointer
    assert e.value.status == ffi.JG_EINVAL
    with pytest.raises(ValueError):
        Tensor.empty((0,), "float16", dev)  # "alloc size must be positve", as the reference's Allocator.alloc
    x9 = Tensor.zeros((65, 64), "float16", dev)
    y9 = Tensor.zeros((65, 16), "float16", dev)
    with pytest.raises(ffi.JgError) as e:
        dev.call("jg_linear", y9.ptr, x9.ptr, w.ptr, 0, 0, 65, 16, 64)  # more rows than one projection call takes
    assert e.value.status == ffi.JG_ENOTSUP
    with pytest.raises(ffi.JgError) as e:  # the fused-norm entry points want pre-normalised rows above 8
        dev.call("jg_norm_linear", y9.ptr, x9.ptr, w.ptr, 1e-5, w.ptr, 0, 9, 16, 64)
    assert e.value.status == ffi.JG_ENOTSUP and "normalise" in str(e.value)
    with pytest.raises(ffi.JgError) as e:
        h = C.c_void_p()
        ffi.call("jg_device_open", 99, C.byref(h))
    assert e.value.status == ffi.JG_EINVAL
    dev.synchronize()  # the device is still usable
    assert (y.numpy() == 0).all()


# ------------------------------------------------------------------------------------------------ exchanges, one rank
def test_peer_exchange_entry_points_with_a_single_rank(dev):
    """A world of one rank exercises the peer-memory kernels' own arithmetic and argument checks without a second GPU:
    the projection fused with its all-reduce must equal the plain residual projection bit for bit (same kernel, sum
    over one rank), the stand-alone exchange must equal round-and-add, the key reduction is the identity."""
    import ctypes as C
    from denograd_b200.multi import TensorParallel
    tp = TensorParallel(dev, 0, 1, TensorParallel.unique_id())
    rng = np.random.default_rng(77)
    M, N, K = 2, 1027, 2048
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    h0 = rng.standard_normal((M, N)).astype(np.float16)
    xt, wt = Tensor(x, device=dev), Tensor(w, device=dev)
    h = Tensor(h0.copy(), device=dev)
    with pytest.raises(ffi.JgError) as e:  # before the buffers are open
        ffi.call("jg_linear_allreduce_residual", tp.handle, h.ptr, xt.ptr, wt.ptr, 0, M, N, K)
    assert e.value.status == 22
    assert tp.open_peers(lambda mine: [mine])
    ffi.call("jg_linear_allreduce_residual", tp.handle, h.ptr, xt.ptr, wt.ptr, 0, M, N, K)
    ref = Tensor(h0.copy(), device=dev)
    dev.call("jg_linear", ref.ptr, xt.ptr, wt.ptr, 0, ref.ptr, M, N, K)
    assert (h.numpy().view(np.uint16) == ref.numpy().view(np.uint16)).all()
    # twice more: the exchange counter alternates the buffer parity
    for _ in range(2):
        ffi.call("jg_linear_allreduce_residual", tp.handle, h.ptr, xt.ptr, wt.ptr, 0, M, N, K)
        dev.call("jg_linear", ref.ptr, xt.ptr, wt.ptr, 0, ref.ptr, M, N, K)
    assert (h.numpy().view(np.uint16) == ref.numpy().view(np.uint16)).all()
    with pytest.raises(ffi.JgError):  # more than 8 rows
        ffi.call("jg_linear_allreduce_residual", tp.handle, h.ptr, xt.ptr, wt.ptr, 0, 9, N, K)
    # stand-alone sum + residual
    part = rng.standard_normal((5, 777)).astype(np.float32)
    hh0 = rng.standard_normal((5, 777)).astype(np.float16)
    pt, hh = Tensor(part, device=dev), Tensor(hh0.copy(), device=dev)
    ffi.call("jg_peer_allreduce_residual", tp.handle, hh.ptr, pt.ptr, part.size)
    want = (hh0.astype(np.float32) + part.astype(np.float16).astype(np.float32)).astype(np.float16)
    assert (hh.numpy().view(np.uint16) == want.view(np.uint16)).all()
    # keys
    keys = rng.integers(0, 2**63, 7, dtype=np.uint64)
    kt = Tensor(keys.copy(), device=dev)
    ffi.call("jg_peer_allreduce_max_u64", tp.handle, kt.ptr, keys.size)
    assert (kt.numpy() == keys).all()
    dev.synchronize()
    tp.close()  # frees the exchange buffer: a later communicator on this device starts afresh


def test_weights_written_just_before_a_projection_are_seen(dev):
    """A weight matrix filled by one of the library's kernels and used by the very next call, with no synchronisation
    in between: the tensor-core projections, which load weight tiles ahead of their dependency wait, must hold those
    loads back.  The buffer is reused with another seed so that a stale read would show."""
    M, N, K = 6, 256, 1024
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
    xt = Tensor(x, device=dev)
    w = Tensor.empty((N, K), "float16", dev)
    y = Tensor.empty((M, N), "float16", dev)
    for seed in (101, 202, 303):
        dev.call("jg_fill_normal_f16", w.ptr, seed, 0, N * K, 0.05)
        dev.call("jg_linear", y.ptr, xt.ptr, w.ptr, 0, 0, M, N, K)  # 6 rows: tcgen05 kernel
        want = O.linear_f16(x, O.synth_normal_f16(seed, N * K, 0.05).reshape(N, K))
        assert_reduction_close(y.numpy(), want, max_ulp=1, max_frac=0.08, what=f"projection right after fill, seed {seed}")
    # the same with a projection's output used as the next projection's weights
    a = Tensor((rng.standard_normal((N, K)) * 0.05).astype(np.float16), device=dev)
    b = Tensor((rng.standard_normal((K, K)) * 0.05).astype(np.float16), device=dev)
    w2 = Tensor.zeros((N, K), "float16", dev)
    dev.synchronize()
    dev.call("jg_linear", w2.ptr, a.ptr, b.ptr, 0, 0, N, K, K)   # w2 = a . b^T, written by a kernel ...
    dev.call("jg_linear", y.ptr, xt.ptr, w2.ptr, 0, 0, M, N, K)  # ... and read as weights by the next one
    w2_host = w2.numpy()
    assert_reduction_close(y.numpy(), O.linear_f16(x, w2_host), max_ulp=1, max_frac=0.08, what="projection over a fresh output")


def test_rows_mapped_to_a_missing_sequence_are_skipped(dev):
    """A row->sequence entry outside the block table is never followed: the row's K/V are not stored, its attention
    output is left alone, and the cache pages of the real sequences stay as they were."""
    rng = np.random.default_rng(12)
    H, G, hd, B, max_ctx = 4, 2, 64, 2, 128
    kv = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=16)
    freqs = precompute_freqs_cis(hd, 2 * max_ctx, 500000.0, dev)
    stride = (H + 2 * G) * hd
    R = 4
    rows = (rng.standard_normal((R, stride)) * 0.7).astype(np.float16)
    qkv = Tensor(rows.copy(), device=dev)
    pos = Tensor(np.array([0, 0, 1, 1], np.int32), device=dev)
    good = Tensor(np.array([0, 1, 0, 1], np.int32), device=dev)
    bad = Tensor(np.array([0, 7, -1, 1], np.int32), device=dev)  # rows 1 and 2 name sequences that do not exist
    out_good = Tensor.zeros((R, H * hd), "float16", dev)
    dev.call("jg_rope_kvwrite_rows", kv.handle, 0, qkv.ptr, freqs.ptr, freqs.shape[0], pos.ptr, good.ptr, R, H)
    dev.call("jg_attn_rows", kv.handle, 0, out_good.ptr, qkv.ptr, pos.ptr, good.ptr, R, H)
    want = out_good.numpy()
    # second cache, same rows, with the bad map: rows 0 and 3 behave as before, 1 and 2 leave no trace
    kv2 = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=16)
    qkv2 = Tensor(rows.copy(), device=dev)
    sentinel = np.full((R, H * hd), 3.0, np.float16)
    out_bad = Tensor(sentinel.copy(), device=dev)
    dev.call("jg_rope_kvwrite_rows", kv2.handle, 0, qkv2.ptr, freqs.ptr, freqs.shape[0], pos.ptr, bad.ptr, R, H)
    dev.call("jg_attn_rows", kv2.handle, 0, out_bad.ptr, qkv2.ptr, pos.ptr, bad.ptr, R, H)
    got = out_bad.numpy()
    assert (got[0].view(np.uint16) == want[0].view(np.uint16)).all()
    assert (got[1] == 3.0).all() and (got[2] == 3.0).all(), "a skipped row's output was written"
    # row 3 (sequence 1, position 1) now sees a zero K/V at position 0, where row 1 was skipped: compare with the checker
    q_rot = qkv2.numpy()[3, :H * hd].reshape(1, 1, H, hd)
    k_ref = np.zeros((1, max_ctx, G, hd), np.float16)
    v_ref = np.zeros_like(k_ref)
    k_ref[0, 1] = O.rope(rows[3, H * hd:(H + G) * hd].reshape(1, G, hd), freqs.numpy(), [1])[0]
    v_ref[0, 1] = rows[3, (H + G) * hd:].reshape(G, hd)
    assert_reduction_close(got[3:4], O.attention(q_rot, k_ref, v_ref, 1).reshape(1, H * hd), max_ulp=2, max_frac=0.2, what="row after a skipped one")
    # the skipped rows' projections are untouched (Q not rotated)
    assert (qkv2.numpy()[1] == rows[1]).all() and (qkv2.numpy()[2] == rows[2]).all()
    kv.close()
    kv2.close()


def test_int8_dequantised_copy_is_bit_exact(dev):
    """jg_dequant_i8_f16 = Int8Linear's weight.cast(half) * scale, one rounding per element; a projection over the
    copy equals the int8 projection's definition."""
    rng = np.random.default_rng(91)
    N, K, M = 384, 1024, 70
    wq = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sc = (rng.uniform(0.5, 1.5, N) * synth.INT8_SCALE_BASE).astype(np.float16)
    wt, st = Tensor(wq, device=dev), Tensor(sc, device=dev)
    dq = Tensor.empty((N, K), "float16", dev)
    dev.call("jg_dequant_i8_f16", dq.ptr, wt.ptr, st.ptr, N, K)
    want = wq.astype(np.float16) * sc[:, None]
    assert (dq.numpy().view(np.uint16) == want.view(np.uint16)).all()
    x = rng.standard_normal((M, K)).astype(np.float16)
    xt = Tensor(x, device=dev)
    y = Tensor.empty((M, N), "float16", dev)
    dev.call("jg_linear", y.ptr, xt.ptr, dq.ptr, 0, 0, M, N, K)  # 70 rows: tcgen05 kernel on the fp16 copy
    assert_reduction_close(y.numpy(), O.linear_w8(x, wq, sc), max_ulp=1, max_frac=0.08, what="projection over the dequantised copy")
    with pytest.raises(ffi.JgError):
        dev.call("jg_dequant_i8_f16", dq.ptr, wt.ptr, st.ptr, N, K + 8)
    dev.synchronize()
