// Device, allocator, timing and graph entry points of libjsgrad_cuda (the Compiled / Allocator / GraphRunner
// side of the boundary; see include/jsgrad_cuda.h for the reference interfaces each one stands in for).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_err[512] = "";

void jg_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int jg_cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  const char* base = strrchr(file, '/');
  jg_set_error("CUDA error %d (%s) at %s:%d in `%s`", (int)e, cudaGetErrorString(e), base ? base + 1 : file, line, what);
  return e == cudaErrorMemoryAllocation ? JG_ENOMEM : JG_EIO;
}

JG_API const char* jg_last_error(void) { return g_err; }

int g_jg_capturing = 0;
static struct { void (*fn)(void*); void* p; } g_deferred[1024];
static int g_n_deferred = 0;

void jg_defer(void (*fn)(void*), void* p) {
  if (g_n_deferred < 1024) { g_deferred[g_n_deferred].fn = fn; g_deferred[g_n_deferred].p = p; g_n_deferred++; }
  // a full queue leaks the object rather than break the capture
}
void jg_run_deferred(void) {
  if (g_jg_capturing > 0) return;
  const int n = g_n_deferred;
  g_n_deferred = 0;
  for (int i = 0; i < n; i++) g_deferred[i].fn(g_deferred[i].p);
}

JG_API int jg_device_count(int32_t* out) {
  JG_REQUIRE(out != nullptr, "null output pointer");
  int n = 0;
  JG_CUDA(cudaGetDeviceCount(&n));
  *out = n;
  return JG_OK;
}

JG_API int jg_device_open(int32_t ordinal, jg_dev** out) {
  JG_REQUIRE(out != nullptr, "null output pointer");
  int n = 0;
  JG_CUDA(cudaGetDeviceCount(&n));
  JG_REQUIRE(ordinal >= 0 && ordinal < n, "device ordinal %d out of range (%d CUDA devices)", ordinal, n);
  JG_CUDA(cudaSetDevice(ordinal));
  jg_dev* d = new jg_dev();
  memset(d, 0, sizeof(*d));
  d->ordinal = ordinal;
  JG_CUDA(cudaGetDeviceProperties(&d->prop, ordinal));
  if (d->prop.major < 10) {
    jg_set_error("device %d is sm_%d%d; this library carries sm_100a code only", ordinal, d->prop.major, d->prop.minor);
    delete d;
    return JG_ENOTSUP;
  }
  d->sm_count = d->prop.multiProcessorCount;
  const char* pdl = getenv("JG_PDL");
  d->pdl = !(pdl && pdl[0] == '0');
  // Thread-block-cluster launches do better without the attribute (8B decode step: 3.256 -> 3.242 ms without it on the
  // attention launches, 3.563 -> 3.426 ms under tensor parallelism without it on attention and the gathering projections):
  // off unless asked for
  const char* pc = getenv("JG_PDL_CLUSTER");
  d->pdl_cluster = (pc && pc[0] == '1');
  const char* pa = getenv("JG_PDL_ATTN");
  d->pdl_attn = (pa && pa[0] == '1');
  JG_CUDA(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  JG_CUDA(cudaEventCreate(&d->t0));
  JG_CUDA(cudaEventCreate(&d->t1));
  d->pinned_stage_bytes = 1 << 16;
  JG_CUDA(cudaHostAlloc(&d->pinned_stage, d->pinned_stage_bytes, cudaHostAllocDefault));
  *out = d;
  return JG_OK;
}

JG_API int jg_device_close(jg_dev* dev) {
  JG_ENTER(dev);
  cudaStreamSynchronize(dev->stream);
  cudaEventDestroy(dev->t0);
  cudaEventDestroy(dev->t1);
  cudaFreeHost(dev->pinned_stage);
  cudaStreamDestroy(dev->stream);
  delete dev;
  return JG_OK;
}

int jg_peer_error(jg_dev* dev, int* code);  // comm.cu
int jg_peer_run_boundary(jg_dev* dev);      // comm.cu: fold the exchange ordinals into the device-resident base

int jg_check_device_errors(jg_dev* dev) {
  if (dev->capturing) return JG_OK;
  if (dev->peer_pending) {
    dev->peer_pending = false;
    int pc = 0;
    int rc = jg_peer_error(dev, &pc);
    if (rc) return rc;
    if (pc != 0) {
      jg_set_error("a peer-memory reduction gave up waiting for another rank's flag; results since the last "
                   "synchronisation are invalid");
      return JG_ETIMEDOUT;
    }
  }
  if (!dev->tc_pending || dev->err_word == nullptr) return JG_OK;
  dev->tc_pending = false;
  int code = 0;
  JG_CUDA(cudaMemcpy(&code, dev->err_word, sizeof(int), cudaMemcpyDeviceToHost));
  if (code != 0) {
    cudaMemset(dev->err_word, 0, sizeof(int));
    jg_set_error("a device-side wait gave up (code %d: 1 = TMA producer, 2 = MMA issuer, 3 = epilogue of a tensor-core "
                 "projection, 4 = grid barrier of the single-kernel decode step); results since the last synchronisation "
                 "are invalid", code);
    return JG_ETIMEDOUT;
  }
  return JG_OK;
}

JG_API int jg_device_sync(jg_dev* dev) {
  JG_ENTER(dev);
  JG_CUDA(cudaStreamSynchronize(dev->stream));
  jg_clear_fresh(dev);
  return jg_check_device_errors(dev);
}

JG_API int jg_device_props(jg_dev* dev, jg_props* out) {
  JG_ENTER(dev);
  JG_REQUIRE(out != nullptr, "null output pointer");
  memset(out, 0, sizeof(*out));
  strncpy(out->name, dev->prop.name, sizeof(out->name) - 1);
  out->sm_count = dev->prop.multiProcessorCount;
  out->cc_major = dev->prop.major;
  out->cc_minor = dev->prop.minor;
  out->total_mem = dev->prop.totalGlobalMem;
  out->l2_bytes = (uint64_t)dev->prop.l2CacheSize;
  out->max_smem_per_block = (int32_t)dev->prop.sharedMemPerBlockOptin;
  return JG_OK;
}

JG_API int jg_launch_count(jg_dev* dev, uint64_t* out) {
  JG_REQUIRE(dev != nullptr && out != nullptr, "null argument");
  *out = dev->launches;
  return JG_OK;
}

// ------------------------------------------------------------------------------------------------ allocator
JG_API int jg_alloc(jg_dev* dev, size_t nbytes, uint64_t* dptr) {
  JG_ENTER(dev);
  JG_REQUIRE(dptr != nullptr, "null output pointer");
  JG_REQUIRE(nbytes > 0, "alloc size must be positive, getting %zu", nbytes);
  JG_REQUIRE(!dev->capturing, "allocation while a graph is being captured");
  void* p = nullptr;
  JG_CUDA(cudaMalloc(&p, nbytes));
  *dptr = (uint64_t)(uintptr_t)p;
  return JG_OK;
}

JG_API int jg_free(jg_dev* dev, uint64_t dptr) {
  JG_ENTER(dev);
  if (dptr == 0) return JG_OK;
  if (g_jg_capturing > 0) { jg_defer([](void* p) { cudaFree(p); }, (void*)(uintptr_t)dptr); return JG_OK; }
  JG_CUDA(cudaStreamSynchronize(dev->stream));
  JG_CUDA(cudaFree((void*)(uintptr_t)dptr));
  return JG_OK;
}

JG_API int jg_copyin(jg_dev* dev, uint64_t dst, const void* host, size_t nbytes) {
  JG_ENTER(dev);
  if (nbytes == 0) return JG_OK;
  JG_REQUIRE(dst != 0 && host != nullptr, "null pointer in copyin");
  JG_REQUIRE(!dev->capturing, "host copy while a graph is being captured");
  // Pageable source: cudaMemcpyAsync stages it before returning, so the caller may reuse `host` at once, and
  // the copy is still ordered after earlier launches on the stream.
  JG_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, host, nbytes, cudaMemcpyHostToDevice, dev->stream));
  // a pinned source would make the call truly asynchronous; callers of this entry point may not keep `host` alive
  JG_CUDA(cudaStreamSynchronize(dev->stream));
  jg_clear_fresh(dev);
  return JG_OK;
}

JG_API int jg_copyout(jg_dev* dev, void* host, uint64_t src, size_t nbytes) {
  JG_ENTER(dev);
  if (nbytes == 0) return JG_OK;
  JG_REQUIRE(src != 0 && host != nullptr, "null pointer in copyout");
  JG_REQUIRE(!dev->capturing, "host copy while a graph is being captured");
  JG_CUDA(cudaMemcpyAsync(host, (const void*)(uintptr_t)src, nbytes, cudaMemcpyDeviceToHost, dev->stream));
  JG_CUDA(cudaStreamSynchronize(dev->stream));
  jg_clear_fresh(dev);
  return jg_check_device_errors(dev);
}

JG_API int jg_copyin_async(jg_dev* dev, uint64_t dst, const void* pinned_host, size_t nbytes) {
  JG_ENTER(dev);
  if (nbytes == 0) return JG_OK;
  JG_REQUIRE(dst != 0 && pinned_host != nullptr, "null pointer in copyin_async");
  JG_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, pinned_host, nbytes, cudaMemcpyHostToDevice, dev->stream));
  jg_mark_fresh(dev, dst, nbytes);
  return JG_OK;
}

JG_API int jg_copyout_async(jg_dev* dev, void* pinned_host, uint64_t src, size_t nbytes) {
  JG_ENTER(dev);
  if (nbytes == 0) return JG_OK;
  JG_REQUIRE(src != 0 && pinned_host != nullptr, "null pointer in copyout_async");
  JG_CUDA(cudaMemcpyAsync(pinned_host, (const void*)(uintptr_t)src, nbytes, cudaMemcpyDeviceToHost, dev->stream));
  return JG_OK;
}

JG_API int jg_transfer(jg_dev* dst_dev, uint64_t dst, jg_dev* src_dev, uint64_t src, size_t nbytes) {
  JG_REQUIRE(dst_dev != nullptr && src_dev != nullptr, "null device handle");
  if (nbytes == 0) return JG_OK;
  JG_REQUIRE(dst != 0 && src != 0, "null pointer in transfer");
  JG_CUDA(cudaSetDevice(src_dev->ordinal));
  // order the copy after the producer's work, run it on the consumer's stream
  cudaEvent_t ev;
  JG_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  JG_CUDA(cudaEventRecord(ev, src_dev->stream));
  JG_CUDA(cudaSetDevice(dst_dev->ordinal));
  JG_CUDA(cudaStreamWaitEvent(dst_dev->stream, ev, 0));
  JG_CUDA(cudaMemcpyPeerAsync((void*)(uintptr_t)dst, dst_dev->ordinal, (const void*)(uintptr_t)src, src_dev->ordinal,
                              nbytes, dst_dev->stream));
  JG_CUDA(cudaEventDestroy(ev));
  return JG_OK;
}

JG_API int jg_memset(jg_dev* dev, uint64_t dst, int32_t byte, size_t nbytes) {
  JG_ENTER(dev);
  if (nbytes == 0) return JG_OK;
  JG_REQUIRE(dst != 0, "null pointer in memset");
  JG_CUDA(cudaMemsetAsync((void*)(uintptr_t)dst, byte, nbytes, dev->stream));
  jg_mark_fresh(dev, dst, nbytes);
  return JG_OK;
}

JG_API int jg_copy(jg_dev* dev, uint64_t dst, uint64_t src, size_t nbytes) {
  JG_ENTER(dev);
  if (nbytes == 0) return JG_OK;
  JG_REQUIRE(dst != 0 && src != 0, "null pointer in copy");
  JG_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, (const void*)(uintptr_t)src, nbytes, cudaMemcpyDeviceToDevice, dev->stream));
  jg_mark_fresh(dev, dst, nbytes);
  return JG_OK;
}

JG_API int jg_host_alloc(size_t nbytes, void** out) {
  JG_REQUIRE(out != nullptr && nbytes > 0, "bad argument to host_alloc");
  JG_CUDA(cudaHostAlloc(out, nbytes, cudaHostAllocDefault));
  return JG_OK;
}

static void host_free_now(void* p) { cudaFreeHost(p); }

JG_API int jg_host_free(void* p) {
  if (!p) return JG_OK;
  if (g_jg_capturing > 0) { jg_defer(host_free_now, p); return JG_OK; }
  JG_CUDA(cudaFreeHost(p));
  return JG_OK;
}

// ------------------------------------------------------------------------------------------------ timing
JG_API int jg_timer_start(jg_dev* dev) {
  JG_ENTER(dev);
  JG_CUDA(cudaEventRecord(dev->t0, dev->stream));
  return JG_OK;
}

JG_API int jg_timer_stop(jg_dev* dev, double* seconds) {
  JG_ENTER(dev);
  JG_REQUIRE(seconds != nullptr, "null output pointer");
  JG_CUDA(cudaEventRecord(dev->t1, dev->stream));
  JG_CUDA(cudaEventSynchronize(dev->t1));
  jg_clear_fresh(dev);
  float ms = 0.f;
  JG_CUDA(cudaEventElapsedTime(&ms, dev->t0, dev->t1));
  *seconds = (double)ms * 1e-3;
  return JG_OK;
}

// ------------------------------------------------------------------------------------------------ graphs
JG_API int jg_graph_begin(jg_dev* dev) {
  JG_ENTER(dev);
  JG_REQUIRE(!dev->capturing, "graph capture already in progress");
  int prc = jg_peer_run_boundary(dev);  // the captured list numbers its peer exchanges from 1
  if (prc) return prc;
  JG_CUDA(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
  dev->capturing = true;
  g_jg_capturing++;
  dev->capture_launches = 0;
  return JG_OK;
}

JG_API int jg_graph_end(jg_dev* dev, jg_graph** out) {
  JG_ENTER(dev);
  JG_REQUIRE(out != nullptr, "null output pointer");
  JG_REQUIRE(dev->capturing, "no graph capture in progress");
  int prc = jg_peer_run_boundary(dev);  // last captured launch: a replay moves the exchange base on by what it holds
  dev->capturing = false;
  g_jg_capturing--;
  cudaGraph_t g = nullptr;
  JG_CUDA(cudaStreamEndCapture(dev->stream, &g));
  if (prc) { cudaGraphDestroy(g); return prc; }
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(g);
    return jg_cuda_fail(e, "cudaGraphInstantiate", __FILE__, __LINE__);
  }
  jg_graph* gr = new jg_graph();
  gr->graph = g;
  gr->exec = exec;
  gr->n_kernels = dev->capture_launches;
  *out = gr;
  jg_run_deferred();
  return JG_OK;
}

JG_API int jg_graph_launch(jg_dev* dev, jg_graph* g) {
  JG_ENTER(dev);
  JG_REQUIRE(g != nullptr && g->exec != nullptr, "null graph");
  JG_REQUIRE(!dev->capturing, "graph launch during capture");
  JG_CUDA(cudaGraphLaunch(g->exec, dev->stream));
  dev->launches += g->n_kernels;
  return JG_OK;
}

static void graph_destroy_now(void* p) {
  jg_graph* g = (jg_graph*)p;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
}

JG_API int jg_graph_destroy(jg_graph* g) {
  if (!g) return JG_OK;
  if (g_jg_capturing > 0) { jg_defer(graph_destroy_now, g); return JG_OK; }
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return JG_OK;
}
