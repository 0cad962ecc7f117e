"""GPU test of jg_attn_decode_noalloc, the decode-attention entry point that allocates nothing.

Hosts whose own allocator owns the device (jsgrad's memory planner hands out every buffer) or that cannot take the
synchronisation of cudaMalloc need a variant whose scratch is part of the library image.  The test drives it through
the C ABI with caller-owned K/V pools, block table, positions, queries and output, and checks that it returns exactly
what jg_attn_decode returns for the same cache contents — twice in a row, with different contexts, because the second
call finds the first call's leftovers in the shared scratch array.  Collected last on purpose: it is the newest entry
point, so a run that stops at the first failure has already exercised everything else.
"""
import numpy as np
import pytest

from denograd_b200 import ffi
from denograd_b200.device import Tensor
from denograd_b200.llama import KVCache

pytestmark = pytest.mark.gpu


def test_noalloc_attention_matches_the_allocating_entry_point(dev):
    rng = np.random.default_rng(7)
    B, H, G, hd, page, max_ctx, n_split = 2, 8, 2, 64, 16, 512, 4
    pages = max_ctx // page
    stride = (H + 2 * G) * hd
    # RoPE table of identities (cos 1, sin 0): jg_rope_kvwrite then stores K exactly as given, so the caller-owned
    # pools below can be written from the same host arrays
    ident = np.zeros((max_ctx, hd // 2, 2), np.float16)
    ident[..., 0] = 1.0
    table = Tensor(ident, device=dev)
    kv = KVCache(dev, 1, H, G, hd, max_ctx, B, page_size=page, n_split=n_split)
    k_pool = np.zeros((B * pages, G, page, hd), np.float16)  # identity block table: row b owns pages [b*pages, ...)
    v_pool = np.zeros_like(k_pool)
    bt = (np.arange(B * pages, dtype=np.int32)).reshape(B, pages)
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
                k_pool[b * pages + t // page, :, t % page] = row[b, H * hd:(H + G) * hd].reshape(G, hd)
                v_pool[b * pages + t // page, :, t % page] = row[b, (H + G) * hd:].reshape(G, hd)
        T_done = T
        kt, vt = Tensor(k_pool, device=dev), Tensor(v_pool, device=dev)
        dev.call("jg_attn_decode", kv.handle, 0, out_ref.ptr, qkv.ptr, pos.ptr, B, H)
        dev.call("jg_attn_decode_noalloc", out_new.ptr, qkv.ptr, kt.ptr, vt.ptr, bt_dev.ptr, pos.ptr, B, H, G, hd, page,
                 pages, n_split)
        ref, new = out_ref.numpy(), out_new.numpy()
        assert np.isfinite(new.astype(np.float32)).all() and np.abs(new.astype(np.float32)).max() > 0
        assert (new.view(np.uint16) == ref.view(np.uint16)).all(), f"context {T}: outputs differ"
    # a shape whose scratch exceeds the built-in array is refused with a clear message, before any launch
    with pytest.raises(ffi.JgError) as e:
        dev.call("jg_attn_decode_noalloc", out_new.ptr, qkv.ptr, kt.ptr, vt.ptr, bt_dev.ptr, pos.ptr, B, H, G, hd, page,
                 1 << 16, n_split)
    assert e.value.status == ffi.JG_EINVAL and "scratch" in str(e.value)
    kv.close()
