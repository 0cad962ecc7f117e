"""Run-time compiled kernels on the device (jg_program_load / jg_program_call): source in the shape the reference's
CUDARenderer emits is compiled, loaded and launched over global_size x local_size with buffers first and int variables
last (the argument order of jsgrad/runtime/ops_clang.ts:44-52); results against numpy.  Integer results are exact;
the fp16 kernel's tolerance is one rounding of the product (it multiplies in fp32 and rounds once, as numpy does)."""
import numpy as np
import pytest

from denograd_b200 import ffi
from denograd_b200.device import CUDACompiler, CUDAGraph, CUDAProgram, Tensor
from tests.test_program import RENDERED

pytestmark = pytest.mark.gpu

REDUCE = """
extern "C" __global__ void __launch_bounds__(128) r_rows_128(float* data0, const float* data1, const int cols) {
  __shared__ float temp0[128];
  int gidx0 = blockIdx.x; /* rows */
  int gidx1 = blockIdx.y; /* 2 */
  int lidx0 = threadIdx.x; /* 128 */
  float acc0 = 0.0f;
  for (int ridx0 = lidx0; ridx0 < cols; ridx0 += 128) { acc0 += data1[(gidx1*gridDim.x+gidx0)*cols+ridx0]; }
  temp0[lidx0] = acc0;
  __syncthreads();
  if (lidx0 == 0) {
    float acc1 = 0.0f;
    for (int ridx1 = 0; ridx1 < 128; ridx1++) { acc1 += temp0[ridx1]; }
    data0[gidx1*gridDim.x+gidx0] = acc1;
  }
}
"""

IOTA = """
extern "C" __global__ void __launch_bounds__(32) E_iota(int* data0, const int start, const int step) {
  int i = (blockIdx.z*gridDim.y+blockIdx.y)*gridDim.x*32 + blockIdx.x*32 + threadIdx.x;
  data0[i] = start + step*i;
}
"""


def test_rendered_elementwise_kernel(dev):
    rng = np.random.default_rng(3)
    n4 = 1000  # work items of four halves each
    x = (rng.standard_normal(n4 * 4) * 3).astype(np.float16)
    scale = np.array([0.37], np.float32)
    prg = CUDAProgram(dev, "E_scale_clip_4", CUDACompiler().compile(RENDERED))
    out, xt, st = Tensor.zeros((n4 * 4,), "float16", dev), Tensor(x, device=dev), Tensor(scale, device=dev)
    prg(out, xt, st, global_size=[(n4 + 63) // 64, 1, 1], local_size=[64, 1, 1], vals=[n4])
    want = (x.astype(np.float32) * scale[0]).astype(np.float16)
    assert (out.numpy().view(np.uint16) == want.view(np.uint16)).all()
    prg.close()


def test_shared_memory_reduce_on_a_2d_grid_and_timing(dev):
    rng = np.random.default_rng(4)
    rows, cols = 37, 1000
    x = rng.integers(-8, 9, (2, rows, cols)).astype(np.float32)  # small integers: every partial sum is exact
    prg = CUDAProgram(dev, "r_rows_128", CUDACompiler().compile(REDUCE))
    out, xt = Tensor.zeros((2, rows), "float32", dev), Tensor(x, device=dev)
    seconds = prg(out, xt, global_size=[rows, 2], local_size=[128], vals=[cols], wait=True)
    assert seconds is not None and 0.0 < seconds < 1.0
    assert (out.numpy() == x.sum(axis=2)).all()


def test_variables_only_3d_grid_graph_replay_and_launch_count(dev):
    prg = CUDAProgram(dev, "E_iota", CUDACompiler().compile(IOTA))
    g = (3, 2, 2)
    n = 32 * g[0] * g[1] * g[2]
    out = Tensor.zeros((n,), "int32", dev)
    before = dev.launch_count()
    prg(out, global_size=g, local_size=(32, 1, 1), vals=[5, 3])
    assert dev.launch_count() == before + 1
    assert (out.numpy() == 5 + 3 * np.arange(n)).all()
    # recorded into a graph like any other launch of the library, replayed with the captured arguments
    out.assign(np.zeros(n, np.int32))
    with CUDAGraph(dev) as graph:
        prg(out, global_size=g, local_size=(32, 1, 1), vals=[-2, 7])
    assert (out.numpy() == 0).all(), "a captured launch must not run"
    graph.launch()
    assert (out.numpy() == -2 + 7 * np.arange(n)).all()


def test_load_and_call_errors(dev):
    lib = CUDACompiler().compile(IOTA)
    with pytest.raises(ffi.JgError) as e:
        CUDAProgram(dev, "no_such_kernel", lib)
    assert e.value.status == ffi.JG_EINVAL and "no_such_kernel" in str(e.value)
    with pytest.raises(ffi.JgError) as e:
        CUDAProgram(dev, "E_iota", b'{"entry": "jg_linear"}')
    assert e.value.status == ffi.JG_EINVAL
    with pytest.raises(ValueError):
        CUDAProgram(dev, "E_iota", b"")
    prg = CUDAProgram(dev, "E_iota", lib)
    out = Tensor.zeros((64,), "int32", dev)
    with pytest.raises(ffi.JgError) as e:  # the kernel was compiled with __launch_bounds__(32)
        prg(out, global_size=[1], local_size=[64], vals=[0, 1])
    assert e.value.status == ffi.JG_EINVAL
    with pytest.raises(ffi.JgError) as e:
        prg(out, global_size=[1, 70000, 1], local_size=[32], vals=[0, 1])
    assert e.value.status == ffi.JG_EINVAL
    prg(out, global_size=[2], local_size=[32], vals=[1, 1])  # the device is still usable
    assert (out.numpy() == 1 + np.arange(64)).all()
