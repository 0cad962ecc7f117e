"""GPU parity of the tcgen05 / TMA projection (3 activation rows and more) against fp32 host arithmetic and, on
sampled rows, against the CPU checker's sequential fp32 accumulation."""
import os
import subprocess
import sys

import numpy as np
import pytest

from denograd_b200.device import Tensor
from oracle import oracle as O
from tests.test_kernels_gpu import assert_reduction_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (65, 256, 512), (200, 384, 1024), (512, 6144, 4096), (300, 4096, 14336),
                                   # few rows: weight streaming with split-K over a cluster (8, 2, 3, 4 CTAs per tile)
                                   (3, 256, 512), (5, 2048, 2048), (9, 256, 512), (16, 4096, 4096), (32, 1024, 14336), (48, 6144, 4096), (64, 4096, 4096),
                                   # gate / up in CTA pairs (tcgen05 cta_group::2), the last tile partly out of range
                                   (512, 4096, 4096), (300, 1024, 512)])
def test_dense_projection_all_epilogues(dev, M, N, K):
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    res = rng.standard_normal((M, N)).astype(np.float16)
    xt, wt, rt = Tensor(x, device=dev), Tensor(w, device=dev), Tensor(res, device=dev)
    y = Tensor.zeros((M, N), "float16", dev)
    acc = x.astype(np.float32) @ w.astype(np.float32).T
    ref = acc.astype(np.float16)
    dev.call("jg_linear", y.ptr, xt.ptr, wt.ptr, 0, 0, M, N, K)
    dev.synchronize()
    got = y.numpy()
    assert_reduction_close(got, ref, max_ulp=1, max_frac=0.08, what=f"tcgen05 linear M{M} N{N} K{K}")
    rows = [0, M // 2, M - 1]  # the checker's own sequential sum on a few rows
    assert_reduction_close(got[rows], O.linear_f16(x[rows], w), max_ulp=1, max_frac=0.08, what="tcgen05 vs checker rows")
    dev.call("jg_linear", y.ptr, xt.ptr, wt.ptr, 0, rt.ptr, M, N, K)
    ref_r = (res.astype(np.float32) + ref.astype(np.float32)).astype(np.float16)
    assert_reduction_close(y.numpy(), ref_r, max_ulp=2, max_frac=0.06, what="tcgen05 linear+residual")
    p32 = Tensor.zeros((M, N), "float32", dev)
    dev.call("jg_linear_partial", p32.ptr, xt.ptr, wt.ptr, 0, M, N, K)
    assert np.abs(p32.numpy() - acc).max() <= 2e-3 * max(1.0, np.abs(acc).max())
    if N <= 4096 and K <= 4096:
        w3 = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
        w3t = Tensor(w3, device=dev)
        dev.call("jg_norm_swiglu", y.ptr, xt.ptr, 0, 1e-5, wt.ptr, 0, w3t.ptr, 0, M, N, K)
        up = (x.astype(np.float32) @ w3.astype(np.float32).T).astype(np.float16)
        assert_reduction_close(y.numpy(), O.swiglu(ref, up), max_ulp=3, max_frac=0.12, what="tcgen05 swiglu")
    dev.synchronize()


def test_cta_pairs_forced_for_every_epilogue():
    """JG_TC_PAIR=2 sends every fp16 projection above 128 rows through the paired kernel (by default only the gate / up
    pair takes it).  The choice is read once per process, hence the child process."""
    pick = "512-6144-4096 or 300-4096-14336 or 512-4096-4096 or 300-1024-512"
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-q", "-x", "-m", "gpu", "-k",
                        f"test_dense_projection_all_epilogues and ({pick})"], env=dict(os.environ, JG_TC_PAIR="2"),
                       capture_output=True, text=True, timeout=900, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "4 passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
