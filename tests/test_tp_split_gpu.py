"""GPU tests of the tensor-parallel exchanges that need no second process: the split all-reduce (a row-parallel
projection pushes, the next projection gathers), the two-shot sum and the single-process communicators.

With one rank the kernels' own arithmetic, buffer parity and argument checks are exercised on one GPU.  With two GPUs in
the box the same entry points run across two devices driven by ONE host thread (the reference engine's threading
model) and are compared with the CPU checker's projection over the unsplit weight matrix."""
import ctypes as C

import numpy as np
import pytest

from denograd_b200 import ffi
from denograd_b200.device import Device, Tensor
from denograd_b200.multi import TensorParallel
from oracle import oracle as O
from tests.test_kernels_gpu import assert_reduction_close

pytestmark = pytest.mark.gpu


def _gpu_count() -> int:
    n = C.c_int32(0)
    try:
        return n.value if ffi.load().jg_device_count(C.byref(n)) == 0 else 0
    except Exception:
        return 0


@pytest.fixture()
def tp1(dev):
    tp = TensorParallel(dev, 0, 1, TensorParallel.unique_id())
    assert tp.open_peers(lambda mine: [mine])
    yield tp
    dev.synchronize()
    tp.close()


@pytest.mark.parametrize("M", [1, 2, 5])
def test_push_then_gather_equals_the_unsplit_block_on_one_rank(dev, tp1, M):
    """wo -> (+residual) -> ffn_norm -> w1/w3 -> SwiGLU and w2 -> (+residual) -> norm -> projection / logits, once
    through the ordinary entry points and once as push + gathering consumer: identical bits, over three rounds so
    that both buffer parities are used."""
    rng = np.random.default_rng(40 + M)
    d, f, V = 512, 768, 1000
    x = (rng.standard_normal((M, d)) * 0.5).astype(np.float16)
    h0 = (rng.standard_normal((M, d)) * 0.5).astype(np.float16)
    wo = (rng.standard_normal((d, d)) * 0.05).astype(np.float16)
    w1 = (rng.standard_normal((f, d)) * 0.05).astype(np.float16)
    w3 = (rng.standard_normal((f, d)) * 0.05).astype(np.float16)
    wv = (rng.standard_normal((V, d)) * 0.05).astype(np.float16)
    g = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float16)
    T = lambda a: Tensor(a, device=dev)
    xt, wot, w1t, w3t, wvt, gt = T(x), T(wo), T(w1), T(w3), T(wv), T(g)
    eps = 1e-5
    for rnd in range(3):
        # reference: the one-device entry points
        h_ref = T(h0.copy())
        dev.call("jg_linear", h_ref.ptr, xt.ptr, wot.ptr, 0, h_ref.ptr, M, d, d)
        y_ref = Tensor.empty((M, f), "float16", dev)
        dev.call("jg_norm_swiglu", y_ref.ptr, h_ref.ptr, gt.ptr, eps, w1t.ptr, 0, w3t.ptr, 0, M, f, d)
        q_ref = Tensor.empty((M, f), "float16", dev)
        dev.call("jg_norm_linear", q_ref.ptr, h_ref.ptr, gt.ptr, eps, w1t.ptr, 0, M, f, d)
        lg_ref, key_ref = Tensor.empty((M, V), "float16", dev), Tensor.zeros((M,), "uint64", dev)
        dev.call("jg_norm_logits_argmax_shard", lg_ref.ptr, key_ref.ptr, h_ref.ptr, gt.ptr, eps, wvt.ptr, 0, M, V, d, 7)
        # split: push, then each of the three consumers
        for kind in ("swiglu", "linear", "logits"):
            h_in, h_out = T(h0.copy()), Tensor.zeros((M, d), "float16", dev)
            ffi.call("jg_tp_linear_push", tp1.handle, xt.ptr, wot.ptr, 0, M, d, d)
            if kind == "swiglu":
                y = Tensor.empty((M, f), "float16", dev)
                ffi.call("jg_tp_norm_swiglu", tp1.handle, y.ptr, h_out.ptr, h_in.ptr, gt.ptr, eps, w1t.ptr, 0, w3t.ptr, 0, M, f, d)
                want = y_ref
            elif kind == "linear":
                y = Tensor.empty((M, f), "float16", dev)
                ffi.call("jg_tp_norm_linear", tp1.handle, y.ptr, h_out.ptr, h_in.ptr, gt.ptr, eps, w1t.ptr, 0, M, f, d)
                want = q_ref
            else:
                y, key = Tensor.empty((M, V), "float16", dev), Tensor.zeros((M,), "uint64", dev)
                ffi.call("jg_tp_norm_logits_argmax", tp1.handle, y.ptr, key.ptr, h_out.ptr, h_in.ptr, gt.ptr, eps, wvt.ptr, 0, M, V, d, 7)
                want = lg_ref
                if M <= 2:
                    assert (key.numpy() == key_ref.numpy()).all()
            if M <= 2:  # the same matrix-vector kernel on both sides: identical bits
                assert (h_out.numpy().view(np.uint16) == h_ref.numpy().view(np.uint16)).all(), (rnd, kind, "residual stream")
                assert (y.numpy().view(np.uint16) == want.numpy().view(np.uint16)).all(), (rnd, kind)
            else:  # from 3 rows on the one-device entry points run on the tensor cores: another summation order
                assert_reduction_close(h_out.numpy(), h_ref.numpy(), max_ulp=1, max_frac=0.08, what=f"residual stream, {kind}")
                assert_reduction_close(y.numpy(), want.numpy(), max_ulp=2, max_frac=0.3, what=kind)
    with pytest.raises(ffi.JgError):  # h_in and h_out must differ
        ffi.call("jg_tp_norm_linear", tp1.handle, y.ptr, h_in.ptr, h_in.ptr, gt.ptr, eps, w1t.ptr, 0, M, f, d)
    with pytest.raises(ffi.JgError):  # more than 8 rows
        ffi.call("jg_tp_linear_push", tp1.handle, xt.ptr, wot.ptr, 0, 9, d, d)
    dev.synchronize()


def test_two_shot_sum_on_one_rank(dev, tp1):
    rng = np.random.default_rng(5)
    rows, d = 37, 512
    part = tp1.partial_tensor(rows, d)
    assert part is not None and part.ptr % 16 == 0
    p = rng.standard_normal((rows, d)).astype(np.float32)
    h0 = rng.standard_normal((rows, d)).astype(np.float16)
    h = Tensor(h0.copy(), device=dev)
    for rnd in range(3):
        part.assign(p)
        tp1.reduce_into_residual(h, part)
        h0 = (h0.astype(np.float32) + p.astype(np.float16).astype(np.float32)).astype(np.float16)
        assert (h.numpy().view(np.uint16) == h0.view(np.uint16)).all(), rnd
    with pytest.raises(ffi.JgError):
        ffi.call("jg_peer_allreduce2_residual", tp1.handle, h.ptr, 6)  # not a multiple of 4
    dev.synchronize()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs 2 GPUs")
def test_one_process_two_devices_against_the_checker():
    """jg_comm_init_all: one host thread drives both ranks.  A row-parallel projection (each device holds half of K)
    through the fused exchange, the split exchange and the two-shot sum, against the checker's projection over the
    whole matrix followed by the fp16 residual add."""
    devs = [Device["CUDA"], Device["CUDA:1"]]
    tps = TensorParallel.init_all(devs)
    assert all(t.peer_capacity > 0 and t.twoshot_capacity > 0 for t in tps)
    rng = np.random.default_rng(77)
    world, N, K = 2, 384, 1024
    Kl = K // world
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    g = (1.0 + 0.1 * rng.standard_normal(N)).astype(np.float16)
    w_next = (rng.standard_normal((256, N)) * 0.05).astype(np.float16)
    for M in (1, 2):
        x = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
        h0 = (rng.standard_normal((M, N)) * 0.5).astype(np.float16)
        want_h = (h0.astype(np.float32) + O.linear_f16(x, w).astype(np.float32)).astype(np.float16)
        want_y = O.linear_f16(O.rmsnorm(want_h, g, 1e-5), w_next)
        xs = [Tensor(np.ascontiguousarray(x[:, r * Kl:(r + 1) * Kl]), device=devs[r]) for r in range(world)]
        ws = [Tensor(np.ascontiguousarray(w[:, r * Kl:(r + 1) * Kl]), device=devs[r]) for r in range(world)]
        # (a) projection fused with the whole exchange
        hs = [Tensor(h0.copy(), device=devs[r]) for r in range(world)]
        for r in range(world):
            ffi.call("jg_linear_allreduce_residual", tps[r].handle, hs[r].ptr, xs[r].ptr, ws[r].ptr, 0, M, N, Kl)
        got = [t.numpy() for t in hs]
        assert (got[0].view(np.uint16) == got[1].view(np.uint16)).all(), "ranks disagree"
        assert_reduction_close(got[0], want_h, max_ulp=1, max_frac=0.08, what="fused exchange")
        # (b) push, then the next norm + projection gathers
        gs = [Tensor(g, device=devs[r]) for r in range(world)]
        wn = [Tensor(w_next, device=devs[r]) for r in range(world)]
        h_in = [Tensor(h0.copy(), device=devs[r]) for r in range(world)]
        h_out = [Tensor.zeros((M, N), "float16", devs[r]) for r in range(world)]
        ys = [Tensor.empty((M, 256), "float16", devs[r]) for r in range(world)]
        for r in range(world):
            ffi.call("jg_tp_linear_push", tps[r].handle, xs[r].ptr, ws[r].ptr, 0, M, N, Kl)
        for r in range(world):
            ffi.call("jg_tp_norm_linear", tps[r].handle, ys[r].ptr, h_out[r].ptr, h_in[r].ptr, gs[r].ptr, 1e-5, wn[r].ptr, 0, M, 256, N)
        got = [t.numpy() for t in h_out]
        assert (got[0].view(np.uint16) == got[1].view(np.uint16)).all(), "ranks disagree"
        assert_reduction_close(got[0], want_h, max_ulp=1, max_frac=0.08, what="split exchange: residual stream")
        assert_reduction_close(ys[0].numpy(), want_y, max_ulp=2, max_frac=0.25, what="split exchange: next projection")
    # (c) two-shot sum of 48 rows
    M = 48
    x = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
    h0 = (rng.standard_normal((M, N)) * 0.5).astype(np.float16)
    want_h = (h0.astype(np.float32) + O.linear_f16(x, w).astype(np.float32)).astype(np.float16)
    hs = [Tensor(h0.copy(), device=devs[r]) for r in range(world)]
    parts = [tps[r].partial_tensor(M, N) for r in range(world)]
    for r in range(world):
        xr = Tensor(np.ascontiguousarray(x[:, r * Kl:(r + 1) * Kl]), device=devs[r])
        wr = Tensor(np.ascontiguousarray(w[:, r * Kl:(r + 1) * Kl]), device=devs[r])
        devs[r].call("jg_linear_partial", parts[r].ptr, xr.ptr, wr.ptr, 0, M, N, Kl)
    for r in range(world):
        tps[r].reduce_into_residual(hs[r], parts[r])
    got = [t.numpy() for t in hs]
    assert (got[0].view(np.uint16) == got[1].view(np.uint16)).all(), "ranks disagree"
    assert_reduction_close(got[0], want_h, max_ulp=1, max_frac=0.08, what="two-shot exchange")
    for d_ in devs:
        d_.synchronize()
    for t in tps:
        t.close()
