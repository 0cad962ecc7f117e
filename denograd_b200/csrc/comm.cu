// Tensor-parallel communicator: one rank per process and GPU, NCCL over NVLink / NVSwitch.
//
// The reference declares a sharding plan (jsgrad/models/llama3.ts:239-249) but its multi-device layer is a stub
// (jsgrad/multi.ts:4-61: every function throws), so there is no reference collective to mirror; this file supplies
// the one exchange the plan needs: an all-reduce after each row-parallel projection, plus a max-reduction of the
// packed (value, index) keys for greedy selection over a vocabulary-sharded output layer.
// NCCL is opened at run time (dlopen of the libnccl.so.2 the caller names, normally the one PyTorch ships), so the
// library itself links against nothing but the CUDA runtime.  The collectives are ordinary stream operations: they
// are captured into the decode graph like the kernels around them.
#include <dlfcn.h>
#include <string.h>

#include "common.cuh"
#include "peer.cuh"

// The slice of NCCL's C API used here (nccl.h of NCCL 2.x; the values are ABI-stable).
typedef struct { char internal[128]; } nccl_unique_id;
typedef struct ncclComm* nccl_comm_t;
enum { NCCL_SUM = 0, NCCL_MAX = 2, NCCL_UINT64 = 5, NCCL_FLOAT16 = 6, NCCL_FLOAT32 = 7 };
typedef int (*fn_get_unique_id)(nccl_unique_id*);
typedef int (*fn_comm_init_rank)(nccl_comm_t*, int, nccl_unique_id, int);
typedef int (*fn_comm_destroy)(nccl_comm_t);
typedef int (*fn_all_reduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t);
typedef const char* (*fn_get_error_string)(int);
typedef int (*fn_comm_init_all)(nccl_comm_t*, int, const int*);
typedef int (*fn_group)(void);

static struct {
  void* handle;
  fn_get_unique_id get_unique_id;
  fn_comm_init_rank comm_init_rank;
  fn_comm_destroy comm_destroy;
  fn_all_reduce all_reduce;
  fn_get_error_string get_error_string;
  fn_comm_init_all comm_init_all;  // optional: single-process communicators
  fn_group group_start, group_end;
} g_nccl = {};

struct jg_comm {
  jg_dev* dev;
  nccl_comm_t comm;
  int rank, world;
  bool in_process;  // made by jg_comm_init_all: the peers' buffers are addressed directly, not through IPC handles
};

static int nccl_open(const char* path) {
  if (g_nccl.handle) return JG_OK;
  void* h = dlopen(path && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    jg_set_error("cannot open NCCL (%s): %s", path && path[0] ? path : "libnccl.so.2", dlerror());
    return JG_ENOTSUP;
  }
  g_nccl.get_unique_id = (fn_get_unique_id)dlsym(h, "ncclGetUniqueId");
  g_nccl.comm_init_rank = (fn_comm_init_rank)dlsym(h, "ncclCommInitRank");
  g_nccl.comm_destroy = (fn_comm_destroy)dlsym(h, "ncclCommDestroy");
  g_nccl.all_reduce = (fn_all_reduce)dlsym(h, "ncclAllReduce");
  g_nccl.get_error_string = (fn_get_error_string)dlsym(h, "ncclGetErrorString");
  g_nccl.comm_init_all = (fn_comm_init_all)dlsym(h, "ncclCommInitAll");
  g_nccl.group_start = (fn_group)dlsym(h, "ncclGroupStart");
  g_nccl.group_end = (fn_group)dlsym(h, "ncclGroupEnd");
  if (!g_nccl.get_unique_id || !g_nccl.comm_init_rank || !g_nccl.comm_destroy || !g_nccl.all_reduce || !g_nccl.get_error_string) {
    jg_set_error("the NCCL library lacks one of ncclGetUniqueId / ncclCommInitRank / ncclCommDestroy / ncclAllReduce");
    dlclose(h);
    memset(&g_nccl, 0, sizeof(g_nccl));
    return JG_ENOTSUP;
  }
  g_nccl.handle = h;
  return JG_OK;
}

static int nccl_fail(int rc, const char* what) {
  jg_set_error("NCCL error %d (%s) in %s", rc, g_nccl.get_error_string ? g_nccl.get_error_string(rc) : "?", what);
  return JG_EIO;
}

JG_API int jg_comm_unique_id(const char* nccl_path, void* id128) {
  JG_REQUIRE(id128 != nullptr, "comm_unique_id: null output");
  int rc = nccl_open(nccl_path);
  if (rc) return rc;
  nccl_unique_id id;
  int n = g_nccl.get_unique_id(&id);
  if (n != 0) return nccl_fail(n, "ncclGetUniqueId");
  memcpy(id128, &id, sizeof(id));
  return JG_OK;
}

JG_API int jg_comm_init(jg_dev* dev, const char* nccl_path, const void* id128, int32_t rank, int32_t world, jg_comm** out) {
  JG_ENTER(dev);
  JG_REQUIRE(id128 != nullptr && out != nullptr, "comm_init: null argument");
  JG_REQUIRE(world >= 1 && rank >= 0 && rank < world, "comm_init: rank %d outside a world of %d", rank, world);
  int rc = nccl_open(nccl_path);
  if (rc) return rc;
  nccl_unique_id id;
  memcpy(&id, id128, sizeof(id));
  nccl_comm_t c = nullptr;
  int n = g_nccl.comm_init_rank(&c, world, id, rank);
  if (n != 0) return nccl_fail(n, "ncclCommInitRank");
  jg_comm* cm = new jg_comm();
  cm->dev = dev; cm->comm = c; cm->rank = rank; cm->world = world;
  *out = cm;
  return JG_OK;
}

static void comm_destroy_now(void* p) { jg_comm_destroy((jg_comm*)p); }

static void peer_release(jg_comm* comm);

JG_API int jg_comm_destroy(jg_comm* comm) {
  if (!comm) return JG_OK;
  if (g_jg_capturing > 0) { jg_defer(comm_destroy_now, comm); return JG_OK; }
  cudaSetDevice(comm->dev->ordinal);
  cudaStreamSynchronize(comm->dev->stream);
  peer_release(comm);  // unmap the peers' exchange buffers, free this rank's own
  if (g_nccl.comm_destroy && comm->comm) g_nccl.comm_destroy(comm->comm);
  delete comm;
  return JG_OK;
}

// In-place sum of `count` fp32 values over the ranks (the partial products of a row-parallel projection).
JG_API int jg_allreduce_sum_f32(jg_comm* comm, uint64_t buf, uint64_t count) {
  JG_REQUIRE(comm != nullptr, "allreduce: null communicator");
  JG_ENTER(comm->dev);
  JG_REQUIRE(count > 0 && jg_aligned(buf, 4), "allreduce_sum_f32: bad buffer");
  if (comm->world == 1) return JG_OK;
  JG_REQUIRE(comm->comm != nullptr, "allreduce_sum_f32: this communicator has no NCCL side");
  int n = g_nccl.all_reduce((const void*)buf, (void*)buf, (size_t)count, NCCL_FLOAT32, NCCL_SUM, comm->comm, comm->dev->stream);
  if (n != 0) return nccl_fail(n, "ncclAllReduce(sum, f32)");
  return JG_OK;
}

// In-place maximum of `count` uint64 keys over the ranks: with keys packed as (ordered fp16 value << 32 | ~index) the
// result is the largest logit and, among equals, the lowest vocabulary index (jsgrad/tensor.ts:2314-2320).
JG_API int jg_allreduce_max_u64(jg_comm* comm, uint64_t buf, uint64_t count) {
  JG_REQUIRE(comm != nullptr, "allreduce: null communicator");
  JG_ENTER(comm->dev);
  JG_REQUIRE(count > 0 && jg_aligned(buf, 8), "allreduce_max_u64: bad buffer");
  if (comm->world == 1) return JG_OK;
  JG_REQUIRE(comm->comm != nullptr, "allreduce_max_u64: this communicator has no NCCL side");
  int n = g_nccl.all_reduce((const void*)buf, (void*)buf, (size_t)count, NCCL_UINT64, NCCL_MAX, comm->comm, comm->dev->stream);
  if (n != 0) return nccl_fail(n, "ncclAllReduce(max, u64)");
  return JG_OK;
}

// ------------------------------------------------------------------------------------------------ peer-memory reductions
// A decode step at small batch all-reduces 16 KB twice per layer; a library collective spends most of that in launch
// and protocol latency.  The exchanges below run over NVLink peer memory (plain cudaMalloc buffers opened through CUDA
// IPC handles; plain stores and loads only).  Sums use flag-in-data entries (peer.cuh): every rank stores each of its
// fp32 partial sums, paired with the exchange number, straight into its slot of every peer's buffer with one 8-byte
// store, then reads the peers' entries from its own buffer, waiting (bounded) until each carries the current exchange
// number — no fence, no separate flag, one NVLink crossing of latency — adds them in rank order (the same order on
// every rank, so all ranks hold bit-identical sums) and applies the residual add of TransformerBlock.call
// (jsgrad/models/llama.ts:125-126) in the same pass.  gemv.cu runs the same exchange inside the projection kernel for
// up to 8 rows (jg_linear_allreduce_residual).  The max-reduction of the greedy keys uses data + one flag per peer.
// Exchanges are numbered 1, 2, 3, ... identically on every rank.  The number is a device word (exchanges completed
// before the current run of launches) plus the launch's ordinal within the run, which the host counts; the word is
// advanced by a one-thread kernel that the library inserts at the borders of a graph capture (the whole run's count is
// added at the end of the captured list, so every replay moves on by as many exchanges as it contains).  No kernel
// spends a fence and an atomic on advancing a counter, and the number is known before the dependency wait.
// Buffers alternate between the two parities of the exchange number: a rank can be at most one exchange ahead of a peer (it needs that peer's entries of the current exchange
// to finish it, and the peer writes them only after its previous exchange has completed), so the slots a slow peer is
// still reading are never overwritten.
struct jg_peer {
  unsigned char* local;                   // this rank's buffer: slots [2][world][PEER_SLOT_FLOATS], then the flags
  unsigned char* mapped[PEER_MAX_WORLD];  // every rank's buffer as mapped here (own entry = local)
  uint32_t* epoch;                        // [0] exchanges completed before the current run of launches (device word)
  uint32_t pending;                       // exchanges launched in the current run (host count)
  int* err;                               // device word: 0 = fine, 1 = a wait for a peer's flag ran out
  unsigned long long timeout_ns;
  bool open;
  bool ipc[PEER_MAX_WORLD];               // mapped[r] came from cudaIpcOpenMemHandle and must be closed
};
static jg_peer g_peer[64] = {};  // by device ordinal

// Undo jg_comm_peer_export / jg_comm_peer_open for this communicator's device: close the IPC mappings, free the
// buffer and the counters, and leave the slot ready for a later communicator.  The stream is idle (caller synchronised).
static void peer_release(jg_comm* comm) {
  const int o = comm->dev->ordinal;
  if (o < 0 || o >= 64) return;
  jg_peer& p = g_peer[o];
  for (int r = 0; r < PEER_MAX_WORLD; r++) {
    if (p.mapped[r] != nullptr && p.ipc[r]) cudaIpcCloseMemHandle(p.mapped[r]);
    p.mapped[r] = nullptr;
    p.ipc[r] = false;
  }
  if (p.local) cudaFree(p.local);
  if (p.epoch) cudaFree(p.epoch);
  cudaGetLastError();
  p = jg_peer{};
}

// h <- h + half(sum over ranks of part): flag-in-data exchange, every thread carries its own elements through it.
__global__ void __launch_bounds__(256) peer_sum_residual_kernel(const PeerArgs a) {
  pdl_launch();
  pdl_wait();
  const uint32_t epoch = a.epoch[0] + a.ord;
  const int parity = (int)(epoch & 1u);
  const long long stride = (long long)gridDim.x * blockDim.x, first = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (long long i = first; i < a.n; i += stride) {
    const float v = a.part[i];
    for (int p = 0; p < a.world; p++)
      if (p != a.rank) peer_ll_store(peer_ll(a.buf[p], parity, a.rank) + i, v, epoch);
  }
  bool ok = true;
  for (long long i = first; i < a.n && ok; i += stride) {
    float sum = 0.f;
    for (int r = 0; r < a.world && ok; r++) {  // rank order on every rank
      float v = a.part[i];
      if (r != a.rank) ok = peer_ll_load(peer_ll(a.buf[a.rank], parity, r) + i, epoch, a.timeout_ns, &v);
      sum = __fadd_rn(sum, v);
    }
    if (ok) a.h[i] = hadd1(a.h[i], __float2half_rn(sum));
  }
  if (!ok) atomicCAS(a.err, 0, 1);
}

// keys <- max over ranks of keys (u64): data into the upper half of every peer's slot, one flag per peer, bounded wait.
__global__ void __launch_bounds__(256) peer_max_kernel(const PeerArgs a) {
  __shared__ int s_fail;
  const int tid = threadIdx.x;
  pdl_launch();
  const uint32_t epoch = a.epoch[0] + a.ord;
  pdl_wait();
  const int parity = (int)(epoch & 1u);
  if (tid == 0) s_fail = 0;
  for (long long i = tid; i < a.n; i += blockDim.x) {
    const unsigned long long v = a.keys[i];
    for (int p = 0; p < a.world; p++)
      if (p != a.rank) reinterpret_cast<unsigned long long*>(peer_slot_hi(a.buf[p], parity, a.rank))[i] = v;
  }
  __syncthreads();  // the release below is cumulative over what this CTA's threads stored before the barrier
  if (tid < a.world && tid != a.rank) {
    uint32_t* f = peer_flag(a.buf[tid], parity, 0, a.rank);
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    const uint32_t* mine = peer_flag(a.buf[a.rank], parity, 0, tid);
    const unsigned long long t0 = global_ns();
    for (;;) {
      uint32_t v;
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (global_ns() - t0 > a.timeout_ns) { s_fail = 1; atomicCAS(a.err, 0, 1); break; }
    }
    asm volatile("fence.acquire.sys;" ::: "memory");
  }
  __syncthreads();
  if (!s_fail) {
    for (long long i = tid; i < a.n; i += blockDim.x) {
      unsigned long long best = a.keys[i];
      for (int r = 0; r < a.world; r++) {
        if (r == a.rank) continue;
        const unsigned long long v = reinterpret_cast<const unsigned long long*>(peer_slot_hi(a.buf[a.rank], parity, r))[i];
        best = v > best ? v : best;
      }
      a.keys[i] = best;
    }
  }
}

// h <- h + half(sum over ranks of partial), two-shot: for messages too large for every rank to send everything to
// everybody.  Rank r owns the r-th slice of the n values.  Each CTA (i) tells the same CTA of every peer that this
// rank's partial sums are complete — they were written by the preceding kernel, into the region of the exchange
// buffer the peers can read — and waits (bounded) for the same word from them; (ii) reads its part of this rank's
// slice from every rank's partial region with plain peer loads, adds them in rank order, rounds once, adds the
// residual, stores the new h and sends it to every peer as flag-in-data entries of (two halves, exchange number);
// (iii) collects the other slices from the entries the peers sent.  One NVLink round trip for the reads plus one
// crossing for the results, n * 4 / world bytes in and n * 2 bytes out per rank.
__global__ void __launch_bounds__(256) peer_sum2_residual_kernel(const PeerArgs a) {
  __shared__ int s_fail;
  const int tid = threadIdx.x, cta = blockIdx.x, nct = gridDim.x;
  pdl_launch();
  const uint32_t epoch = a.epoch[0] + a.ord;
  pdl_wait();
  const int parity = (int)(epoch & 1u);
  const int rank = a.rank, world = a.world;
  if (tid == 0) s_fail = 0;
  __syncthreads();
  // (i) hand-shake with CTA `cta` of every peer
  if (tid < world && tid != rank) {
    uint32_t* f = peer_flag(a.buf[tid], parity, cta, rank);
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    const uint32_t* mine = peer_flag(a.buf[rank], parity, cta, tid);
    const unsigned long long t0 = global_ns();
    for (;;) {
      uint32_t v;
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (global_ns() - t0 > a.timeout_ns) { s_fail = 1; atomicCAS(a.err, 0, 1); break; }
    }
    asm volatile("fence.acquire.sys;" ::: "memory");
  }
  __syncthreads();
  const long long quads = a.n / 4;                                  // 4 values = one 16-byte peer load, two result entries
  const long long per_rank = (quads + world - 1) / world;           // slice of a rank, in quads
  const long long per_cta = (per_rank + nct - 1) / nct;             // part of a slice handled by one CTA
  if (!s_fail) {
    // (ii) this rank's slice
    const long long q_lo = rank * per_rank + (long long)cta * per_cta;
    const long long q_hi = min(min(q_lo + per_cta, (long long)(rank + 1) * per_rank), quads);
    for (long long q = q_lo + tid; q < q_hi; q += blockDim.x) {
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; r++) {  // rank order on every rank
        const float4* src = reinterpret_cast<const float4*>(peer_partial(a.buf[r])) + q;
        float4 v;
        asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(src) : "memory");
        sum.x = __fadd_rn(sum.x, v.x); sum.y = __fadd_rn(sum.y, v.y); sum.z = __fadd_rn(sum.z, v.z); sum.w = __fadd_rn(sum.w, v.w);
      }
      uint2 raw = reinterpret_cast<const uint2*>(a.h)[q];
      __half* hh = reinterpret_cast<__half*>(&raw);
      hh[0] = hadd1(hh[0], __float2half_rn(sum.x)); hh[1] = hadd1(hh[1], __float2half_rn(sum.y));
      hh[2] = hadd1(hh[2], __float2half_rn(sum.z)); hh[3] = hadd1(hh[3], __float2half_rn(sum.w));
      reinterpret_cast<uint2*>(a.h)[q] = raw;
      for (int p = 0; p < world; p++) {
        if (p == rank) continue;
        uint2* dst = peer_result(a.buf[p], parity) + 2 * q;
        peer_ll_store_bits(dst, raw.x, epoch);
        peer_ll_store_bits(dst + 1, raw.y, epoch);
      }
    }
    // (iii) the other ranks' slices, from the entries they sent
    bool ok = true;
    for (int r = 0; r < world && ok; r++) {
      if (r == rank) continue;
      const long long o_lo = r * per_rank + (long long)cta * per_cta;
      const long long o_hi = min(min(o_lo + per_cta, (long long)(r + 1) * per_rank), quads);
      for (long long q = o_lo + tid; q < o_hi && ok; q += blockDim.x) {
        float b0, b1;
        ok = peer_ll_load2(peer_result(a.buf[rank], parity) + 2 * q, epoch, a.timeout_ns, &b0, &b1);
        if (ok) reinterpret_cast<uint2*>(a.h)[q] = make_uint2(__float_as_uint(b0), __float_as_uint(b1));
      }
    }
    if (!ok) atomicCAS(a.err, 0, 1);
  }
}

// Allocate this rank's exchange buffer and return its 64-byte CUDA IPC handle, to be handed to every other rank.
JG_API int jg_comm_peer_export(jg_comm* comm, void* handle64) {
  JG_REQUIRE(comm != nullptr && handle64 != nullptr, "comm_peer_export: null argument");
  JG_ENTER(comm->dev);
  JG_REQUIRE(comm->world <= PEER_MAX_WORLD, "comm_peer_export: at most %d ranks", PEER_MAX_WORLD);
  JG_REQUIRE(!comm->in_process, "comm_peer_export: communicators made by jg_comm_init_all have their buffers already");
  JG_REQUIRE(comm->dev->ordinal >= 0 && comm->dev->ordinal < 64, "comm_peer_export: device ordinal out of range");
  JG_REQUIRE(!comm->dev->capturing, "comm_peer_export: not inside a graph capture");
  jg_peer& p = g_peer[comm->dev->ordinal];
  if (p.local == nullptr) {
    JG_CUDA(cudaMalloc(&p.local, PEER_BYTES));
    JG_CUDA(cudaMemset(p.local, 0, PEER_BYTES));
    JG_CUDA(cudaMalloc(&p.epoch, PEER_MAX_CTAS * sizeof(uint32_t) + sizeof(int)));
    JG_CUDA(cudaMemset(p.epoch, 0, PEER_MAX_CTAS * sizeof(uint32_t) + sizeof(int)));
    p.err = reinterpret_cast<int*>(p.epoch + PEER_MAX_CTAS);
    const char* e = getenv("JG_PEER_TIMEOUT_MS");
    p.timeout_ns = (unsigned long long)(e ? atoll(e) : 5000) * 1000000ull;
  }
  cudaIpcMemHandle_t h;
  JG_CUDA(cudaIpcGetMemHandle(&h, p.local));
  static_assert(sizeof(h) == 64, "CUDA IPC handle size");
  memcpy(handle64, &h, sizeof(h));
  return JG_OK;
}

// Open the other ranks' buffers: handles = world x 64 bytes in rank order (this rank's own entry is ignored).
JG_API int jg_comm_peer_open(jg_comm* comm, const void* handles) {
  JG_REQUIRE(comm != nullptr && handles != nullptr, "comm_peer_open: null argument");
  JG_ENTER(comm->dev);
  jg_peer& p = g_peer[comm->dev->ordinal];
  JG_REQUIRE(p.local != nullptr, "comm_peer_open: call jg_comm_peer_export first");
  JG_REQUIRE(!comm->dev->capturing, "comm_peer_open: not inside a graph capture");
  for (int r = 0; r < comm->world; r++) {
    if (r == comm->rank) { p.mapped[r] = p.local; p.ipc[r] = false; continue; }
    if (p.mapped[r] != nullptr && p.ipc[r]) { cudaIpcCloseMemHandle(p.mapped[r]); p.mapped[r] = nullptr; }  // an earlier communicator's
    cudaIpcMemHandle_t h;
    memcpy(&h, (const unsigned char*)handles + (size_t)r * 64, sizeof(h));
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      jg_set_error("comm_peer_open: rank %d's buffer cannot be mapped (%s); the NCCL path remains available", r, cudaGetErrorString(e));
      return JG_ENOTSUP;
    }
    p.mapped[r] = (unsigned char*)ptr;
    p.ipc[r] = true;
  }
  p.open = true;
  return JG_OK;
}

// Largest element count jg_peer_allreduce_residual takes (0 = the peer path is not open on this communicator's device).
JG_API int jg_comm_peer_capacity(jg_comm* comm, uint64_t* floats) {
  JG_REQUIRE(comm != nullptr && floats != nullptr, "comm_peer_capacity: null argument");
  const int o = comm->dev->ordinal;
  *floats = (o >= 0 && o < 64 && g_peer[o].open) ? PEER_LL_VALUES : 0;
  return JG_OK;
}

int jg_peer_fill_args(jg_comm* comm, PeerArgs* a, bool consume) {
  jg_dev* dev = comm->dev;
  JG_REQUIRE(dev->ordinal >= 0 && dev->ordinal < 64 && g_peer[dev->ordinal].open,
             "peer reduction: the peer buffers are not open (jg_comm_peer_export / jg_comm_peer_open)");
  jg_peer& p = g_peer[dev->ordinal];
  JG_REQUIRE(!consume || p.pending > 0, "peer reduction: nothing has been pushed that this call could gather");
  for (int r = 0; r < comm->world; r++) a->buf[r] = p.mapped[r];
  a->epoch = p.epoch; a->err = p.err; a->timeout_ns = p.timeout_ns; a->rank = comm->rank; a->world = comm->world;
  a->ord = consume ? p.pending : ++p.pending;
  dev->peer_pending = true;
  return JG_OK;
}

// The same for a launch that makes `count` exchanges itself (the single-kernel decode step): a->ord is the first of them.
int jg_peer_fill_args_n(jg_comm* comm, PeerArgs* a, uint32_t count) {
  JG_REQUIRE(comm != nullptr && count > 0, "peer exchange: null communicator or no exchanges");
  int rc = jg_peer_fill_args(comm, a, false);
  if (rc) return rc;
  g_peer[comm->dev->ordinal].pending += count - 1;
  return JG_OK;
}

// One thread: the exchanges of the run that ends here are done; later launches number theirs from the new base.
__global__ void peer_advance_kernel(uint32_t* base, uint32_t n) {
  pdl_launch();
  pdl_wait();
  base[0] += n;
}

// Called by jg_graph_begin (before the capture starts) and jg_graph_end (as the last captured launch): fold the
// exchanges launched so far into the device word, so that a captured list starts from ordinal 1 and every replay
// advances the word by the number of exchanges it holds.
int jg_peer_run_boundary(jg_dev* dev) {
  if (dev->ordinal < 0 || dev->ordinal >= 64) return JG_OK;
  jg_peer& p = g_peer[dev->ordinal];
  if (p.epoch == nullptr || p.pending == 0) return JG_OK;
  const uint32_t n = p.pending;
  p.pending = 0;
  return jg_launch(dev, "peer_advance", peer_advance_kernel, dim3(1), dim3(1), 0, p.epoch, n);
}

static int peer_launch(jg_comm* comm, int mode, uint64_t h, uint64_t part, uint64_t keys, long long n) {
  jg_dev* dev = comm->dev;
  PeerArgs a = {};
  int rc = jg_peer_fill_args(comm, &a);
  if (rc) return rc;
  a.part = (const float*)part; a.h = (__half*)h; a.keys = (unsigned long long*)keys; a.n = n;
  if (mode == 0) {
    int ctas = (int)((n + 1023) / 1024);
    if (ctas > 32) ctas = 32;
    return jg_launch(dev, "peer_allreduce_residual", peer_sum_residual_kernel, dim3(ctas), dim3(256), 0, a);
  }
  if (mode == 2) {
    // one quad per thread in step (ii) when the slice allows it; at most 64 CTAs (one flag row each)
    const long long per_rank = (n / 4 + comm->world - 1) / comm->world;
    int ctas = (int)((per_rank + 255) / 256);
    if (ctas > 64) ctas = 64;
    if (ctas < 1) ctas = 1;
    return jg_launch(dev, "peer_allreduce2_residual", peer_sum2_residual_kernel, dim3(ctas), dim3(256), 0, a);
  }
  return jg_launch(dev, "peer_allreduce_max", peer_max_kernel, dim3(1), dim3(256), 0, a);
}

// h[i] <- h[i] + half( sum over ranks of part[i] ), i < n: all-reduce of a row-parallel projection's fp32 partial sums
// fused with the residual add.  Every rank must make the same sequence of peer reductions with the same n.
JG_API int jg_peer_allreduce_residual(jg_comm* comm, uint64_t h, uint64_t part32, uint64_t n) {
  JG_REQUIRE(comm != nullptr, "peer_allreduce_residual: null communicator");
  JG_ENTER(comm->dev);
  JG_REQUIRE(n > 0 && n <= PEER_LL_VALUES, "peer_allreduce_residual: n=%llu must be at most %llu", (unsigned long long)n,
             (unsigned long long)PEER_LL_VALUES);
  JG_REQUIRE(jg_aligned(h, 2) && jg_aligned(part32, 4), "peer_allreduce_residual: null or misaligned pointer");
  return peer_launch(comm, 0, h, part32, 0, (long long)n);
}

// Where this rank's fp32 partial sums must be written (by jg_linear_partial) for jg_peer_allreduce2_residual: a region
// of the exchange buffer the peers read directly.  floats = its capacity.
JG_API int jg_comm_peer_partial(jg_comm* comm, uint64_t* ptr, uint64_t* floats) {
  JG_REQUIRE(comm != nullptr && ptr != nullptr && floats != nullptr, "comm_peer_partial: null argument");
  const int o = comm->dev->ordinal;
  JG_REQUIRE(o >= 0 && o < 64 && g_peer[o].open, "comm_peer_partial: the peer buffers are not open");
  *ptr = (uint64_t)(uintptr_t)(g_peer[o].local + PEER_PARTIAL_OFFSET);
  *floats = PEER_TWOSHOT_VALUES;
  return JG_OK;
}

// h[i] <- h[i] + half( sum over ranks of partial[i] ), i < n, where every rank's partial sums lie in its
// jg_comm_peer_partial region (two-shot exchange: each rank reduces 1/world of the values and sends the results).
JG_API int jg_peer_allreduce2_residual(jg_comm* comm, uint64_t h, uint64_t n) {
  JG_REQUIRE(comm != nullptr, "peer_allreduce2_residual: null communicator");
  JG_ENTER(comm->dev);
  JG_REQUIRE(n > 0 && n % 4 == 0 && n <= PEER_TWOSHOT_VALUES, "peer_allreduce2_residual: n=%llu must be a multiple of 4, at most %llu",
             (unsigned long long)n, (unsigned long long)PEER_TWOSHOT_VALUES);
  JG_REQUIRE(jg_aligned(h, 8), "peer_allreduce2_residual: null or misaligned pointer");
  return peer_launch(comm, 2, h, 0, 0, (long long)n);
}

// keys[i] <- max over ranks of keys[i] (packed greedy keys of a vocabulary-sharded output layer).
JG_API int jg_peer_allreduce_max_u64(jg_comm* comm, uint64_t keys, uint64_t n) {
  JG_REQUIRE(comm != nullptr, "peer_allreduce_max_u64: null communicator");
  JG_ENTER(comm->dev);
  JG_REQUIRE(n > 0 && n * 4 <= PEER_SLOT_FLOATS, "peer_allreduce_max_u64: n=%llu out of range", (unsigned long long)n);
  JG_REQUIRE(jg_aligned(keys, 8), "peer_allreduce_max_u64: null or misaligned pointer");
  return peer_launch(comm, 1, 0, 0, keys, (long long)n);
}

jg_dev* jg_comm_device(jg_comm* comm) { return comm ? comm->dev : nullptr; }

// Device error word of the peer reductions for jg_check_device_errors (0 = none recorded).
int jg_peer_error(jg_dev* dev, int* code) {
  *code = 0;
  if (dev->ordinal < 0 || dev->ordinal >= 64 || g_peer[dev->ordinal].err == nullptr) return JG_OK;
  JG_CUDA(cudaMemcpy(code, g_peer[dev->ordinal].err, sizeof(int), cudaMemcpyDeviceToHost));
  if (*code) JG_CUDA(cudaMemset(g_peer[dev->ordinal].err, 0, sizeof(int)));
  return JG_OK;
}

// ------------------------------------------------------------------------------------------------ one process, N devices
// All ranks of a tensor-parallel group in ONE process (the reference engine is a single thread that drives every
// device, jsgrad/tensor.ts:676-687): devs[r] becomes rank r.  The exchange buffers are allocated here and addressed
// directly after cudaDeviceEnablePeerAccess, so neither a unique id nor IPC handles travel anywhere;
// jg_comm_peer_export / jg_comm_peer_open are not needed (and not allowed) on these communicators.  The peer-memory
// exchanges work as with one process per rank: a kernel that waits for its peers does so on its own GPU while the host
// thread goes on to launch the peers' kernels.  NCCL collectives issued rank after rank by one thread must be
// bracketed by jg_comm_group_begin / jg_comm_group_end.
JG_API int jg_comm_init_all(int32_t n, jg_dev** devs, const char* nccl_path, jg_comm** out) {
  JG_REQUIRE(devs != nullptr && out != nullptr && n >= 1 && n <= PEER_MAX_WORLD, "comm_init_all: 1..%d devices", PEER_MAX_WORLD);
  for (int r = 0; r < n; r++) {
    JG_REQUIRE(devs[r] != nullptr && devs[r]->ordinal >= 0 && devs[r]->ordinal < 64, "comm_init_all: bad device %d", r);
    JG_REQUIRE(!devs[r]->capturing, "comm_init_all: not inside a graph capture");
    JG_REQUIRE(g_peer[devs[r]->ordinal].local == nullptr, "comm_init_all: device %d already has an exchange buffer", devs[r]->ordinal);
    for (int q = 0; q < r; q++) JG_REQUIRE(devs[q]->ordinal != devs[r]->ordinal, "comm_init_all: device %d listed twice", devs[r]->ordinal);
  }
  nccl_comm_t nc[PEER_MAX_WORLD] = {};
  bool have_nccl = false;
  if (n > 1 && nccl_open(nccl_path) == JG_OK && g_nccl.comm_init_all) {
    int ords[PEER_MAX_WORLD];
    for (int r = 0; r < n; r++) ords[r] = devs[r]->ordinal;
    const int rc = g_nccl.comm_init_all(nc, n, ords);
    if (rc != 0) return nccl_fail(rc, "ncclCommInitAll");
    have_nccl = true;
  }
  // exchange buffers + peer access in both directions
  for (int r = 0; r < n; r++) {
    JG_CUDA(cudaSetDevice(devs[r]->ordinal));
    jg_peer& p = g_peer[devs[r]->ordinal];
    JG_CUDA(cudaMalloc(&p.local, PEER_BYTES));
    JG_CUDA(cudaMemset(p.local, 0, PEER_BYTES));
    JG_CUDA(cudaMalloc(&p.epoch, PEER_MAX_CTAS * sizeof(uint32_t) + sizeof(int)));
    JG_CUDA(cudaMemset(p.epoch, 0, PEER_MAX_CTAS * sizeof(uint32_t) + sizeof(int)));
    p.err = reinterpret_cast<int*>(p.epoch + PEER_MAX_CTAS);
    const char* e = getenv("JG_PEER_TIMEOUT_MS");
    p.timeout_ns = (unsigned long long)(e ? atoll(e) : 5000) * 1000000ull;
    for (int q = 0; q < n; q++) {
      if (q == r) continue;
      int can = 0;
      JG_CUDA(cudaDeviceCanAccessPeer(&can, devs[r]->ordinal, devs[q]->ordinal));
      if (!can) { jg_set_error("comm_init_all: device %d cannot address device %d's memory", devs[r]->ordinal, devs[q]->ordinal); return JG_ENOTSUP; }
      cudaError_t pe = cudaDeviceEnablePeerAccess(devs[q]->ordinal, 0);
      if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) return jg_cuda_fail(pe, "cudaDeviceEnablePeerAccess", __FILE__, __LINE__);
      cudaGetLastError();
    }
  }
  for (int r = 0; r < n; r++) {
    jg_peer& p = g_peer[devs[r]->ordinal];
    for (int q = 0; q < n; q++) { p.mapped[q] = g_peer[devs[q]->ordinal].local; p.ipc[q] = false; }
    p.open = true;
    jg_comm* cm = new jg_comm();
    cm->dev = devs[r]; cm->comm = have_nccl ? nc[r] : nullptr; cm->rank = r; cm->world = n; cm->in_process = true;
    out[r] = cm;
  }
  return JG_OK;
}

// ncclGroupStart / ncclGroupEnd: one thread issuing the same NCCL collective for several ranks must bracket them.
JG_API int jg_comm_group_begin(void) {
  if (!g_nccl.group_start) return JG_OK;
  const int rc = g_nccl.group_start();
  return rc == 0 ? JG_OK : nccl_fail(rc, "ncclGroupStart");
}
JG_API int jg_comm_group_end(void) {
  if (!g_nccl.group_end) return JG_OK;
  const int rc = g_nccl.group_end();
  return rc == 0 ? JG_OK : nccl_fail(rc, "ncclGroupEnd");
}

