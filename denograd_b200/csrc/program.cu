// Run-time compiled kernels: the Compiler / Program pair of a jsgrad device (jsgrad/runtime/allocator.ts:98-107 Program,
// :121-139 CompileError / Compiler; jsgrad/runtime/ops_clang.ts:7-54 is the reference's own instance of the pair) for CUDA C source.
// The reference ships the code generator — CUDARenderer, jsgrad/renderer/cstyle.ts:348-419: `extern "C" __global__ void
// __launch_bounds__(n) name(T* data0, const T* data1, ..., const int var0, ...)`, blockIdx / threadIdx for the global /
// local work-item ids — but no CUDA runtime to hand its output to.  This file is that runtime: source -> cubin through
// NVRTC, cubin -> function through the driver's module API, and a launch of (buffers..., int variables...) over
// global_size x local_size on the device's stream.  It is the path of every AST the hand-written kernels of this
// library do not cover; nothing on the Llama path goes through it.
//
// NVRTC is opened at first use (dlopen), so the library has no link-time dependency on it and a host without it loses
// only this file's entry points (JG_ENOTSUP with the names that were tried).
#include <cuda.h>
#include <dlfcn.h>
#include <nvrtc.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "common.cuh"

namespace {

struct Nvrtc {
  void* so = nullptr;
  nvrtcResult (*create)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  nvrtcResult (*compile)(nvrtcProgram, int, const char* const*) = nullptr;
  nvrtcResult (*destroy)(nvrtcProgram*) = nullptr;
  nvrtcResult (*cubin_size)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*cubin)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*log_size)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*log)(nvrtcProgram, char*) = nullptr;
  const char* (*error_string)(nvrtcResult) = nullptr;
  std::string tried;
};

std::string cuda_home() {
  for (const char* v : {"JSGRAD_CUDA_HOME", "CUDA_HOME", "CUDA_PATH"}) {
    const char* e = getenv(v);
    if (e && *e) return e;
  }
  return "/usr/local/cuda";
}

Nvrtc* nvrtc() {
  static Nvrtc n;
  static bool done = false;
  if (done) return &n;
  done = true;
  std::vector<std::string> names;
  if (const char* e = getenv("JSGRAD_NVRTC_LIB")) names.push_back(e);
  names.push_back("libnvrtc.so.12");
  names.push_back("libnvrtc.so");
  names.push_back(cuda_home() + "/lib64/libnvrtc.so.12");
  names.push_back(cuda_home() + "/lib64/libnvrtc.so");
  for (const auto& nm : names) {
    n.so = dlopen(nm.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (n.so) break;
    n.tried += (n.tried.empty() ? "" : ", ") + nm;
  }
  if (!n.so) return &n;
  bool ok = true;
  auto sym = [&](const char* s) { void* p = dlsym(n.so, s); ok &= p != nullptr; return p; };
  n.create = (decltype(n.create))sym("nvrtcCreateProgram");
  n.compile = (decltype(n.compile))sym("nvrtcCompileProgram");
  n.destroy = (decltype(n.destroy))sym("nvrtcDestroyProgram");
  n.cubin_size = (decltype(n.cubin_size))sym("nvrtcGetCUBINSize");
  n.cubin = (decltype(n.cubin))sym("nvrtcGetCUBIN");
  n.log_size = (decltype(n.log_size))sym("nvrtcGetProgramLogSize");
  n.log = (decltype(n.log))sym("nvrtcGetProgramLog");
  n.error_string = (decltype(n.error_string))sym("nvrtcGetErrorString");
  if (!ok) { dlclose(n.so); n.so = nullptr; n.tried = "a libnvrtc without the cubin entry points"; }
  return &n;
}

// The driver entry points of the module API, fetched through the runtime (the library links no libcuda).
struct Driver {
  CUresult (*module_load_data)(CUmodule*, const void*) = nullptr;
  CUresult (*module_get_function)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*module_unload)(CUmodule) = nullptr;
  CUresult (*launch_kernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
  CUresult (*func_get_attribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
  bool ok = false;
};

Driver* driver() {
  static Driver d;
  static bool done = false;
  if (done) return d.ok ? &d : nullptr;
  done = true;
  bool ok = true;
  auto get = [&](const char* s) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(s, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) { ok = false; fn = nullptr; }
    return fn;
  };
  d.module_load_data = (decltype(d.module_load_data))get("cuModuleLoadData");
  d.module_get_function = (decltype(d.module_get_function))get("cuModuleGetFunction");
  d.module_unload = (decltype(d.module_unload))get("cuModuleUnload");
  d.launch_kernel = (decltype(d.launch_kernel))get("cuLaunchKernel");
  d.func_get_attribute = (decltype(d.func_get_attribute))get("cuFuncGetAttribute");
  d.ok = ok;
  return ok ? &d : nullptr;
}

}  // namespace

struct jg_program {
  jg_dev* dev;
  CUmodule module;
  CUfunction fn;
  int max_threads;  // the function's own limit (__launch_bounds__, registers)
  std::string name;
};

// Compiler.compile (jsgrad/runtime/allocator.ts:128): CUDA C source -> cubin for `arch` ("sm_100a" when null or empty).
// Needs no device.  A source that does not compile is JG_EINVAL with NVRTC's log as the message — the reference raises
// an error carrying the compiler's output the same way (CompileError, jsgrad/runtime/allocator.ts:121; ops_clang.ts:21).
JG_API int jg_cuda_compile(const char* src, const char* arch, uint8_t** image, uint64_t* size) {
  JG_REQUIRE(src != nullptr && image != nullptr && size != nullptr, "cuda_compile: null argument");
  *image = nullptr;
  *size = 0;
  Nvrtc* n = nvrtc();
  if (!n->so) {
    jg_set_error("cuda_compile: NVRTC could not be opened (tried %s; JSGRAD_NVRTC_LIB names another)", n->tried.c_str());
    return JG_ENOTSUP;
  }
  const std::string a = std::string("--gpu-architecture=") + ((arch && *arch) ? arch : "sm_100a");
  const std::string inc = "--include-path=" + cuda_home() + "/include";
  const char* opts[] = {a.c_str(), inc.c_str(), "--std=c++17"};
  nvrtcProgram prog;
  nvrtcResult r = n->create(&prog, src, "jsgrad_kernel.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) { jg_set_error("cuda_compile: nvrtcCreateProgram: %s", n->error_string(r)); return JG_EIO; }
  r = n->compile(prog, 3, opts);
  if (r != NVRTC_SUCCESS) {
    size_t ls = 0;
    n->log_size(prog, &ls);
    std::string log(ls ? ls : 1, '\0');
    if (ls) n->log(prog, &log[0]);
    n->destroy(&prog);
    jg_set_error("cuda_compile: %s\n%.3000s", n->error_string(r), log.c_str());
    return r == NVRTC_ERROR_COMPILATION ? JG_EINVAL : JG_EIO;
  }
  size_t cs = 0;
  r = n->cubin_size(prog, &cs);
  if (r != NVRTC_SUCCESS || cs == 0) {
    n->destroy(&prog);
    jg_set_error("cuda_compile: no cubin for %s (a virtual architecture was named?)", a.c_str());
    return JG_EINVAL;
  }
  uint8_t* out = (uint8_t*)malloc(cs);
  if (!out) { n->destroy(&prog); jg_set_error("cuda_compile: out of host memory for %zu bytes", cs); return JG_ENOMEM; }
  r = n->cubin(prog, (char*)out);
  n->destroy(&prog);
  if (r != NVRTC_SUCCESS) { free(out); jg_set_error("cuda_compile: nvrtcGetCUBIN: %s", n->error_string(r)); return JG_EIO; }
  *image = out;
  *size = cs;
  return JG_OK;
}

JG_API int jg_cuda_image_free(uint8_t* image) {
  free(image);
  return JG_OK;
}

// Program.init(name, lib) (jsgrad/runtime/allocator.ts:101-103, ops_clang.ts:32-40): `image` is what jg_cuda_compile
// returned (or the same bytes from the engine's compile cache), `name` the kernel's function name.
JG_API int jg_program_load(jg_dev* dev, const char* name, const uint8_t* image, uint64_t size, jg_program** out) {
  JG_ENTER(dev);
  JG_REQUIRE(out != nullptr, "program_load: null output pointer");
  *out = nullptr;
  JG_REQUIRE(name != nullptr && *name, "program_load: the kernel needs a name");  // ops_clang.ts:35
  JG_REQUIRE(image != nullptr && size >= 4, "program_load: the image is empty");   // ops_clang.ts:34
  JG_REQUIRE(memcmp(image, "\x7f" "ELF", 4) == 0, "program_load: the image is not a cubin (no ELF header)");
  JG_REQUIRE(!dev->capturing, "program_load while a graph is being captured");
  Driver* d = driver();
  if (!d) { jg_set_error("program_load: the driver's module API is not available"); return JG_ENOTSUP; }
  JG_CUDA(cudaFree(0));  // the device's primary context exists and is current for the driver calls below
  jg_program* p = new jg_program();
  p->dev = dev;
  p->name = name;
  CUresult r = d->module_load_data(&p->module, image);
  if (r != CUDA_SUCCESS) { delete p; jg_set_error("program_load: cuModuleLoadData failed (%d): an image for another architecture?", (int)r); return JG_EINVAL; }
  r = d->module_get_function(&p->fn, p->module, name);
  if (r != CUDA_SUCCESS) { d->module_unload(p->module); delete p; jg_set_error("program_load: no kernel '%s' in the image (%d)", name, (int)r); return JG_EINVAL; }
  p->max_threads = 1024;
  d->func_get_attribute(&p->max_threads, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, p->fn);
  *out = p;
  return JG_OK;
}

// Program.call(bufs, {global_size, local_size, vals}) (jsgrad/runtime/allocator.ts:98,104-106; argument order as in
// ops_clang.ts:44-52: every buffer as a pointer, then every variable as a 32-bit int).  global_size / local_size are
// three numbers each (null = 1, 1, 1); the launch goes onto the device's stream like every other kernel of the
// library, so it is ordered with them, recorded by a graph capture and timed by jg_timer_start / jg_timer_stop.
JG_API int jg_program_call(jg_program* p, const uint64_t* bufs, int32_t n_bufs, const int32_t* vals, int32_t n_vals,
                           const uint32_t* global_size, const uint32_t* local_size) {
  JG_REQUIRE(p != nullptr, "program_call: null program");
  JG_ENTER(p->dev);
  JG_REQUIRE(n_bufs >= 0 && n_vals >= 0 && n_bufs + n_vals <= 512, "program_call: %d buffers and %d variables", n_bufs, n_vals);
  JG_REQUIRE((n_bufs == 0 || bufs != nullptr) && (n_vals == 0 || vals != nullptr), "program_call: null argument list");
  uint32_t g[3] = {1, 1, 1}, l[3] = {1, 1, 1};
  for (int i = 0; i < 3; i++) {
    if (global_size) g[i] = global_size[i];
    if (local_size) l[i] = local_size[i];
  }
  // the limits CUDARenderer schedules against (cstyle.ts:350-351) and the function's own
  JG_REQUIRE(g[0] >= 1 && g[1] >= 1 && g[2] >= 1 && g[0] <= 2147483647u && g[1] <= 65535u && g[2] <= 65535u,
             "program_call %s: global_size %u x %u x %u outside the grid limits", p->name.c_str(), g[0], g[1], g[2]);
  JG_REQUIRE(l[0] >= 1 && l[1] >= 1 && l[2] >= 1 && l[0] <= 1024u && l[1] <= 1024u && l[2] <= 64u &&
                 (uint64_t)l[0] * l[1] * l[2] <= (uint64_t)p->max_threads,
             "program_call %s: local_size %u x %u x %u exceeds the kernel's %d threads per block", p->name.c_str(), l[0], l[1], l[2], p->max_threads);
  Driver* d = driver();
  if (!d) { jg_set_error("program_call: the driver's module API is not available"); return JG_ENOTSUP; }
  std::vector<uint64_t> bcopy(bufs, bufs + n_bufs);
  std::vector<int32_t> vcopy(vals, vals + n_vals);
  std::vector<void*> params;
  params.reserve(n_bufs + n_vals);
  for (int i = 0; i < n_bufs; i++) params.push_back(&bcopy[i]);
  for (int i = 0; i < n_vals; i++) params.push_back(&vcopy[i]);
  const CUresult r = d->launch_kernel(p->fn, g[0], g[1], g[2], l[0], l[1], l[2], 0, (CUstream)p->dev->stream,
                                      params.empty() ? nullptr : params.data(), nullptr);
  if (r != CUDA_SUCCESS) { jg_set_error("program_call %s: cuLaunchKernel failed (%d)", p->name.c_str(), (int)r); return JG_EIO; }
  if (p->dev->capturing) p->dev->capture_launches++;
  else p->dev->launches++;
  return JG_OK;
}

JG_API int jg_program_destroy(jg_program* p) {
  if (!p) return JG_OK;
  if (g_jg_capturing > 0) {  // unloading synchronises: not during a capture
    jg_defer([](void* q) { jg_program_destroy((jg_program*)q); }, p);
    return JG_OK;
  }
  Driver* d = driver();
  cudaSetDevice(p->dev->ordinal);
  cudaStreamSynchronize(p->dev->stream);
  if (d) d->module_unload(p->module);
  delete p;
  return JG_OK;
}
