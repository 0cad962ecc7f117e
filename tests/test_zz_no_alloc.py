"""GPU test of jg_attn_decode_noalloc, the decode-attention entry point that allocates nothing.

Hosts whose own allocator owns the device (jsgrad's memory planner hands out every buffer) or that cannot take the
synchronisation of cudaMalloc need a variant whose scratch is part of the library image.  The test drives it through
the C ABI with caller-owned K/V pools, a scattered block table, positions, queries and output, and checks the result
two ways — against the CPU checker's attention (an independent computation) and bit for bit against jg_attn_decode on
the same cache contents — twice in a row, with different contexts, because the second call finds the first call's
leftovers in the shared scratch array.  Collected last on purpose: it is the newest entry point, so a run that stops
at the first failure has already exercised everything else.
"""
import numpy as np
import pytest

from denograd_b200 import ffi
from denograd_b200.device import Tensor
from denograd_b200.llama import KVCache
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _ulp_close(got: np.ndarray, ref: np.ndarray) -> None:
    """fp16 results of fp32 reductions summed in another order than the checker's: the suite's common bound."""
    from tests.test_kernels_gpu import assert_reduction_close
    assert_reduction_close(got, ref, max_ulp=2, max_frac=0.10, what="attention without allocation")


@pytest.mark.parametrize("H,G,hd,page", [(8, 2, 64, 16), (16, 2, 128, 32)])
def test_noalloc_attention_matches_checker_and_allocating_entry_point(dev, H, G, hd, page):
    rng = np.random.default_rng(7 + H)
    B, max_ctx, n_split = 2, 512, 4
    pages = max_ctx // page
    n_pages = B * pages
    stride = (H + 2 * G) * hd
    # RoPE table of identities (cos 1, sin 0): jg_rope_kvwrite then stores K exactly as given, so the caller-owned
    # pools below can be written from the same host arrays
    ident = np.zeros((max_ctx, hd // 2, 2), np.float16)
    ident[..., 0] = 1.0
    table = Tensor(ident, device=dev)
    kv = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=page, n_split=n_split)
    bt = rng.permutation(n_pages).astype(np.int32).reshape(B, pages)  # every sequence's pages scattered over the pool
    kv.set_block_table(bt)
    k_pool = np.zeros((n_pages, G, page, hd), np.float16)
    v_pool = np.zeros_like(k_pool)
    k_ref = np.zeros((B, max_ctx, G, hd), np.float16)  # the contiguous cache the checker reads
    v_ref = np.zeros_like(k_ref)
    qkv = Tensor.empty((B, stride), "float16", dev)
    pos = Tensor.zeros((B,), "int32", dev)
    out_ref = Tensor.empty((B, H * hd), "float16", dev)
    out_new = Tensor.empty((B, H * hd), "float16", dev)
    bt_dev = Tensor(bt, device=dev)
    T_done = 0
    for T in (37, 301):  # two calls in a row; the second reuses the scratch the first one dirtied
        for t in range(T_done, T):
            row = (rng.standard_normal((B, stride)) * 0.7).astype(np.float16)
            qkv.assign(row)
            pos.assign(np.full((B,), t, np.int32))
            dev.call("jg_rope_kvwrite", kv.handle, 0, qkv.ptr, table.ptr, max_ctx, pos.ptr, B, H)
            for b in range(B):
                k_ref[b, t] = row[b, H * hd:(H + G) * hd].reshape(G, hd)
                v_ref[b, t] = row[b, (H + G) * hd:].reshape(G, hd)
                k_pool[bt[b, t // page], :, t % page] = k_ref[b, t]
                v_pool[bt[b, t // page], :, t % page] = v_ref[b, t]
        T_done = T
        kt, vt = Tensor(k_pool, device=dev), Tensor(v_pool, device=dev)
        dev.call("jg_attn_decode", kv.handle, 0, out_ref.ptr, qkv.ptr, pos.ptr, B, H)
        dev.call("jg_attn_decode_noalloc", out_new.ptr, qkv.ptr, kt.ptr, vt.ptr, bt_dev.ptr, pos.ptr, B, H, G, hd, page,
                 pages, n_split, n_pages)
        ref, new = out_ref.numpy(), out_new.numpy()
        q = row[:, :H * hd].reshape(B, 1, H, hd)
        want = O.attention(q, k_ref, v_ref, T - 1).reshape(B, H * hd)
        _ulp_close(new, want)
        assert (new.view(np.uint16) == ref.view(np.uint16)).all(), f"context {T}: outputs differ"
    # a block-table entry outside the pool is not followed: that page reads as zeros, like unwritten positions
    bad = bt.copy()
    bad[0, 1] = n_pages + 12345
    bad[1, 0] = -3
    dev.call("jg_attn_decode_noalloc", out_new.ptr, qkv.ptr, kt.ptr, vt.ptr, Tensor(bad, device=dev).ptr, pos.ptr, B, H, G,
             hd, page, pages, n_split, n_pages)
    k_bad, v_bad = k_ref.copy(), v_ref.copy()
    k_bad[0, page:2 * page] = 0; v_bad[0, page:2 * page] = 0
    k_bad[1, 0:page] = 0; v_bad[1, 0:page] = 0
    _ulp_close(out_new.numpy(), O.attention(q, k_bad, v_bad, T - 1).reshape(B, H * hd))
    # a shape whose scratch exceeds the built-in array is refused with a clear message, before any launch
    with pytest.raises(ffi.JgError) as e:
        dev.call("jg_attn_decode_noalloc", out_new.ptr, qkv.ptr, kt.ptr, vt.ptr, bt_dev.ptr, pos.ptr, B, H, G, hd, page,
                 1 << 16, n_split, n_pages)
    assert e.value.status == ffi.JG_EINVAL and "scratch" in str(e.value)
    with pytest.raises(ffi.JgError) as e:  # pages x page size beyond an int
        dev.call("jg_attn_decode_noalloc", out_new.ptr, qkv.ptr, kt.ptr, vt.ptr, bt_dev.ptr, pos.ptr, B, H, G, hd, 64,
                 1 << 26, n_split, n_pages)
    assert e.value.status == ffi.JG_EINVAL
    kv.close()
