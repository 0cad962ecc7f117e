// Shared internals of libjsgrad_cuda: device object, error plumbing, small device helpers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jsgrad_cuda.h"

#define JG_API extern "C" __attribute__((visibility("default")))

struct jg_dev {
  int ordinal;
  cudaStream_t stream;
  cudaDeviceProp prop;
  int sm_count;
  bool capturing;
  uint64_t launches;          // kernels launched (graph replays add their node count)
  uint64_t capture_launches;  // kernels recorded into the graph being captured
  cudaEvent_t t0, t1;
  void* pinned_stage;  // small page-locked staging area for jg_copyin of tiny payloads
  size_t pinned_stage_bytes;
  bool pdl;  // launch kernels with programmatic stream serialization (JG_PDL=0 turns it off)
  bool pdl_cluster;  // ... also the thread-block-cluster launches of the gathering projections (JG_PDL_CLUSTER=1; default off)
  bool pdl_attn;     // ... also the decode-attention cluster launches (JG_PDL_ATTN=1; default off)
  int* err_word;    // device word written by kernels whose bounded waits gave up (0 = fine); allocated on first use
  bool tc_pending;  // such kernels were launched since the word was last checked
  bool peer_pending;  // peer-memory reductions (comm.cu) were launched since their error word was last checked
  // Device ranges written by the library's own launches since the stream was last synchronised (the latest
  // JG_FRESH_RING of them).  The tensor-core projection kernels load weight tiles before they wait for their
  // predecessor — right for parameters that were there all along, wrong for a matrix one of the preceding launches
  // is still writing (a dequantised copy, a seeded fill, a projection output reused as a weight).
  uint64_t fresh_lo[16], fresh_hi[16];
  unsigned fresh_n;
};
int jg_check_device_errors(jg_dev* dev);  // after a stream synchronise: JG_ETIMEDOUT if a bounded wait gave up

struct jg_graph {
  cudaGraph_t graph;
  cudaGraphExec_t exec;
  uint64_t n_kernels;
};

void jg_set_error(const char* fmt, ...);
// Releases that may not run while a stream capture is in progress (cudaFree / cudaFreeHost / a stream synchronise
// invalidate the capture): a host whose garbage collector finalises an object in the middle of a capture gets its
// release queued here and carried out right after jg_graph_end.
extern int g_jg_capturing;  // devices of this process with a capture in progress
void jg_defer(void (*fn)(void*), void* p);
void jg_run_deferred(void);
int jg_cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define JG_CUDA(call)                                                        \
  do {                                                                       \
    cudaError_t _e = (call);                                                 \
    if (_e != cudaSuccess) return jg_cuda_fail(_e, #call, __FILE__, __LINE__); \
  } while (0)

#define JG_REQUIRE(cond, ...)   \
  do {                          \
    if (!(cond)) {              \
      jg_set_error(__VA_ARGS__); \
      return JG_EINVAL;         \
    }                           \
  } while (0)

// Makes `dev` current, and counts + checks a launch.  Used right after every <<<>>>.
static inline int jg_after_launch(jg_dev* dev, const char* name) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return jg_cuda_fail(e, name, __FILE__, __LINE__);
  if (dev->capturing) dev->capture_launches++;
  else dev->launches++;
  return JG_OK;
}
#define JG_ENTER(dev)                                              \
  do {                                                             \
    JG_REQUIRE((dev) != nullptr, "null device handle");            \
    JG_CUDA(cudaSetDevice((dev)->ordinal));                        \
  } while (0)

static inline bool jg_aligned(uint64_t p, uint64_t a) { return p != 0 && (p % a) == 0; }
constexpr unsigned JG_FRESH_RING = 16;
static inline void jg_mark_fresh(jg_dev* dev, uint64_t lo, uint64_t bytes) {
  const unsigned i = dev->fresh_n++ % JG_FRESH_RING;
  dev->fresh_lo[i] = lo;
  dev->fresh_hi[i] = lo + bytes;
}
// After a stream synchronisation nothing is in flight: every earlier write is visible to any later launch.
static inline void jg_clear_fresh(jg_dev* dev) {
  for (unsigned i = 0; i < JG_FRESH_RING; i++) dev->fresh_lo[i] = dev->fresh_hi[i] = 0;
}
// Whether `p` lies in memory a weight-producing kernel wrote recently: such weights must not be read ahead of the
// dependency wait.
static inline bool jg_is_fresh(const jg_dev* dev, const void* p) {
  const uint64_t v = (uint64_t)(uintptr_t)p;
  for (unsigned i = 0; i < JG_FRESH_RING; i++)
    if (v != 0 && v >= dev->fresh_lo[i] && v < dev->fresh_hi[i]) return true;
  return false;
}

#ifdef __CUDACC__
// Every kernel of the library is launched through here.  With `dev->pdl` the launch carries the programmatic
// stream-serialization attribute: the kernel may begin while its predecessor on the stream is still draining, and
// must execute pdl_wait() before it touches anything the predecessor wrote (all kernels here do, at their top or,
// for the weight-streaming kernels, right after their first weight prefetch).
// `cluster_x` > 1 launches thread-block clusters of that many CTAs along x (the grid's x must be a multiple of it).
template <typename... KArgs, typename... Args>
static inline int jg_launch_cluster(jg_dev* dev, const char* name, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster_x > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)cluster_x;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    na++;
  }
  if (dev->pdl && (cluster_x <= 1 || dev->pdl_cluster)) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
  if (e != cudaSuccess) return jg_cuda_fail(e, name, __FILE__, __LINE__);
  return jg_after_launch(dev, name);
}
template <typename... KArgs, typename... Args>
static inline int jg_launch(jg_dev* dev, const char* name, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            Args... args) {
  return jg_launch_cluster(dev, name, kern, grid, block, smem, 1, args...);
}
#endif

// ------------------------------------------------------------------------------------------------ device side
#ifdef __CUDACC__

// Programmatic dependent launch: wait until the preceding kernel on the stream has completed and its writes are
// visible (a no-op when the kernel was launched without the attribute) / allow the next kernel to start launching.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 128-bit streaming load of read-only weights: bypass L1 allocation, they are read exactly once per launch.
__device__ __forceinline__ uint4 ld_stream_128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// 128-bit cached load (activations, KV rows: L1/L2 resident or reused)
__device__ __forceinline__ uint4 ld_128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ float2 h2_to_f2(uint32_t u) {
  __half2 h = *reinterpret_cast<__half2*>(&u);
  return __half22float2(h);
}

// exact fp16 x fp16 products accumulated in fp32 (an FMA of an exact product equals multiply-then-add)
__device__ __forceinline__ float dot8_acc(float acc, const uint4& w, const float (&x)[8]) {
  float2 a = h2_to_f2(w.x), b = h2_to_f2(w.y), c = h2_to_f2(w.z), d = h2_to_f2(w.w);
  acc = fmaf(a.x, x[0], acc); acc = fmaf(a.y, x[1], acc);
  acc = fmaf(b.x, x[2], acc); acc = fmaf(b.y, x[3], acc);
  acc = fmaf(c.x, x[4], acc); acc = fmaf(c.y, x[5], acc);
  acc = fmaf(d.x, x[6], acc); acc = fmaf(d.y, x[7], acc);
  return acc;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), c = h2_to_f2(v.z), d = h2_to_f2(v.w);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// fp16 elementwise ops with exactly one rounding and no contraction into FMA.
__device__ __forceinline__ __half hmul1(__half a, __half b) { return __hmul_rn(a, b); }
__device__ __forceinline__ __half hadd1(__half a, __half b) { return __hadd_rn(a, b); }
__device__ __forceinline__ __half hsub1(__half a, __half b) { return __hsub_rn(a, b); }
__device__ __forceinline__ __half hrecip1(__half a) { return __float2half_rn(__fdiv_rn(1.0f, __half2float(a))); }

// Order-preserving map of fp16 bits to uint16 (larger value -> larger key); NaNs are not expected.
__device__ __forceinline__ uint32_t half_order_key(__half h) {
  uint32_t u = __half_as_ushort(h);
  return (u & 0x8000u) ? (~u & 0xFFFFu) : (u | 0x8000u);
}
// (value, lowest index) packed so that an unsigned max picks the largest value and, among equals, the smallest index
__device__ __forceinline__ unsigned long long argmax_key(__half v, uint32_t idx) {
  return ((unsigned long long)half_order_key(v) << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}
#endif
