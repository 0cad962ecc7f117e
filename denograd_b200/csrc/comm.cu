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

// The slice of NCCL's C API used here (nccl.h of NCCL 2.x; the values are ABI-stable).
typedef struct { char internal[128]; } nccl_unique_id;
typedef struct ncclComm* nccl_comm_t;
enum { NCCL_SUM = 0, NCCL_MAX = 2, NCCL_UINT64 = 5, NCCL_FLOAT16 = 6, NCCL_FLOAT32 = 7 };
typedef int (*fn_get_unique_id)(nccl_unique_id*);
typedef int (*fn_comm_init_rank)(nccl_comm_t*, int, nccl_unique_id, int);
typedef int (*fn_comm_destroy)(nccl_comm_t);
typedef int (*fn_all_reduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t);
typedef const char* (*fn_get_error_string)(int);

static struct {
  void* handle;
  fn_get_unique_id get_unique_id;
  fn_comm_init_rank comm_init_rank;
  fn_comm_destroy comm_destroy;
  fn_all_reduce all_reduce;
  fn_get_error_string get_error_string;
} g_nccl = {};

struct jg_comm {
  jg_dev* dev;
  nccl_comm_t comm;
  int rank, world;
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

JG_API int jg_comm_destroy(jg_comm* comm) {
  if (!comm) return JG_OK;
  if (g_jg_capturing > 0) { jg_defer(comm_destroy_now, comm); return JG_OK; }
  cudaSetDevice(comm->dev->ordinal);
  cudaStreamSynchronize(comm->dev->stream);
  if (g_nccl.comm_destroy) g_nccl.comm_destroy(comm->comm);
  delete comm;
  return JG_OK;
}

// In-place sum of `count` fp32 values over the ranks (the partial products of a row-parallel projection).
JG_API int jg_allreduce_sum_f32(jg_comm* comm, uint64_t buf, uint64_t count) {
  JG_REQUIRE(comm != nullptr, "allreduce: null communicator");
  JG_ENTER(comm->dev);
  JG_REQUIRE(count > 0 && jg_aligned(buf, 4), "allreduce_sum_f32: bad buffer");
  if (comm->world == 1) return JG_OK;
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
  int n = g_nccl.all_reduce((const void*)buf, (void*)buf, (size_t)count, NCCL_UINT64, NCCL_MAX, comm->comm, comm->dev->stream);
  if (n != 0) return nccl_fail(n, "ncclAllReduce(max, u64)");
  return JG_OK;
}
