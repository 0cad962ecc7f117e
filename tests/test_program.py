"""The run-time compiler half of the Compiler / Program pair (jg_cuda_compile), which needs no device: CUDA C in the
shape the reference's CUDARenderer emits (jsgrad/renderer/cstyle.ts:348-419: an INFINITY / NAN prefix, cuda_fp16.h
when halves occur, a vector struct with its make_ function, `extern "C" __global__ void __launch_bounds__(n)
name(buffers..., const int vars...)`) becomes a cubin; a broken source raises with the compiler's log."""
import ctypes as C

import pytest

from denograd_b200 import ffi
from denograd_b200.device import CompileError, CUDACompiler

# A kernel written the way the renderer writes them: one output buffer first, inputs const, a symbolic variable last,
# global / local work-item ids from blockIdx / threadIdx, a half4 vector type introduced by the prefix.
RENDERED = """
#define INFINITY (__int_as_float(0x7f800000))
#define NAN (__int_as_float(0x7fffffff))
#include <cuda_fp16.h>
struct __align__(8) half4 { half x, y, z, w; }; __device__ half4 make_half4(half x, half y, half z, half w) { half4 r={x, y, z, w}; return r; }
extern "C" __global__ void __launch_bounds__(64) E_scale_clip_4(half* data0, const half* data1, const float* data2, const int n) {
  int gidx0 = blockIdx.x; /* blocks */
  int lidx0 = threadIdx.x; /* 64 */
  int alu0 = ((gidx0*64)+lidx0);
  if (alu0 < n) {
    half4 val0 = *((half4*)(data1+(alu0*4)));
    float val1 = data2[0];
    float a = min((float)(val0.x)*val1, INFINITY), b = (float)(val0.y)*val1, c = (float)(val0.z)*val1, d = (float)(val0.w)*val1;
    *((half4*)(data0+(alu0*4))) = make_half4((half)(a), (half)(b), (half)(c), (half)(d));
  }
}
"""


def test_rendered_source_compiles_to_a_cubin():
    lib = CUDACompiler().compile(RENDERED)
    assert lib[:4] == b"\x7fELF" and len(lib) > 1000
    assert b"E_scale_clip_4" in lib


def test_compile_error_carries_the_log():
    with pytest.raises(CompileError) as e:
        CUDACompiler().compile('extern "C" __global__ void k(float* data0) { data0[0] = missing_symbol; }')
    assert "missing_symbol" in str(e.value) and "error" in str(e.value)


def test_compile_cached_compiles_once():
    c = CUDACompiler()
    src = 'extern "C" __global__ void k(float* data0) { data0[threadIdx.x] = 1.0f; }'
    a = c.compile_cached(src)
    assert c.compile_cached(src) is a


def test_other_real_architectures_and_a_virtual_one():
    src = 'extern "C" __global__ void k(int* data0) { data0[0] = 7; }'
    assert CUDACompiler("sm_90").compile(src)[:4] == b"\x7fELF"
    with pytest.raises((CompileError, ffi.JgError)):
        CUDACompiler("compute_100a").compile(src)  # PTX only: there is no cubin to load


def test_null_arguments_are_rejected():
    lib = ffi.load()
    image, size = C.c_void_p(), C.c_uint64()
    assert lib.jg_cuda_compile(None, None, C.byref(image), C.byref(size)) == ffi.JG_EINVAL
    assert lib.jg_cuda_compile(b"", None, None, C.byref(size)) == ffi.JG_EINVAL
    assert lib.jg_cuda_image_free(None) == ffi.JG_OK
    assert lib.jg_program_destroy(None) == ffi.JG_OK
