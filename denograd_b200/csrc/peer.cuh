// Shared between comm.cu (buffers, stand-alone reductions) and gemv.cu (projections fused with one or both halves of
// their all-reduce): layout of a rank's peer-exchange buffer and the device helpers that address it.
#pragma once
#include "common.cuh"

constexpr int PEER_MAX_WORLD = 8;
constexpr int PEER_MAX_CTAS = 512;  // flag rows of the flag-based exchanges (keys, two-shot sums): one flag per CTA and rank
constexpr size_t PEER_SLOT_FLOATS = 128 * 1024;  // 512 KB of fp32 per (parity, rank): larger exchanges go through NCCL
constexpr size_t PEER_FLAG_WORDS = 2 * PEER_MAX_CTAS * PEER_MAX_WORLD;
// Two-shot sums (messages too large for every rank to send everything to everybody): this rank's fp32 partial sums
// live in a region the peers read (one copy, no parity: a rank finishes an exchange only after every peer has read
// its slice of it), and the finished fp16 values come back as flag-in-data entries of (two halves, exchange number).
constexpr size_t PEER_TWOSHOT_VALUES = 256 * 1024;  // 1 MB of fp32 partial sums, e.g. 64 rows x 4096
constexpr size_t PEER_SLOTS_BYTES = 2 * PEER_MAX_WORLD * PEER_SLOT_FLOATS * sizeof(float);
constexpr size_t PEER_FLAGS_OFFSET = PEER_SLOTS_BYTES;
constexpr size_t PEER_RESULT_OFFSET = PEER_FLAGS_OFFSET + PEER_FLAG_WORDS * sizeof(uint32_t);  // [2][VALUES/2] entries of 8 B
constexpr size_t PEER_RESULT_BYTES = 2 * (PEER_TWOSHOT_VALUES / 2) * 8;
constexpr size_t PEER_PARTIAL_OFFSET = PEER_RESULT_OFFSET + PEER_RESULT_BYTES;
constexpr size_t PEER_BYTES = PEER_PARTIAL_OFFSET + PEER_TWOSHOT_VALUES * sizeof(float);

struct PeerArgs {
  unsigned char* buf[PEER_MAX_WORLD];
  const uint32_t* epoch;  // device word: exchanges completed before the current run of launches (see comm.cu)
  uint32_t ord;           // this exchange's number within the run: its exchange number is epoch[0] + ord
  int* err;
  const float* part;  // [n] this rank's partial sums (fp32) / packed keys (as 2 x u32 per key)
  __half* h;          // [n] residual stream, updated in place (sum mode)
  unsigned long long* keys;  // [n] (max mode), updated in place
  long long n;        // floats (sum mode) or keys (max mode)
  unsigned long long timeout_ns;
  int rank, world;
};

__device__ __forceinline__ float* peer_slot(unsigned char* buf, int parity, int r) {
  return reinterpret_cast<float*>(buf) + ((size_t)parity * PEER_MAX_WORLD + r) * PEER_SLOT_FLOATS;
}
__device__ __forceinline__ uint32_t* peer_flag(unsigned char* buf, int parity, int cta, int r) {
  return reinterpret_cast<uint32_t*>(buf + PEER_FLAGS_OFFSET) + ((size_t)parity * PEER_MAX_CTAS + cta) * PEER_MAX_WORLD + r;
}
__device__ __forceinline__ uint2* peer_result(unsigned char* buf, int parity) {
  return reinterpret_cast<uint2*>(buf + PEER_RESULT_OFFSET) + (size_t)parity * (PEER_TWOSHOT_VALUES / 2);
}
__device__ __forceinline__ const float* peer_partial(const unsigned char* buf) {
  return reinterpret_cast<const float*>(buf + PEER_PARTIAL_OFFSET);
}
// Flag-in-data exchange for small sums: the lower half of a slot holds up to PEER_LL_VALUES entries of
// (value bits, exchange number), each written with one 8-byte store, so a receiver that sees the right exchange number
// has the value — no fence and no separate flag.  Flag-based exchanges (keys) use the upper half of the slot.
constexpr size_t PEER_LL_VALUES = PEER_SLOT_FLOATS / 4;  // 32 K entries = 256 KB
__device__ __forceinline__ uint2* peer_ll(unsigned char* buf, int parity, int r) {
  return reinterpret_cast<uint2*>(peer_slot(buf, parity, r));
}
__device__ __forceinline__ float* peer_slot_hi(unsigned char* buf, int parity, int r) {
  return peer_slot(buf, parity, r) + PEER_SLOT_FLOATS / 2;
}
__device__ __forceinline__ void peer_ll_store(uint2* p, float v, uint32_t epoch) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ void peer_ll_store_bits(uint2* p, uint32_t bits, uint32_t epoch) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(bits), "r"(epoch) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns();
// Wait (bounded) until entry *p carries `epoch`; false = gave up.
__device__ __forceinline__ bool peer_ll_load(const uint2* p, uint32_t epoch, unsigned long long timeout_ns, float* out) {
  uint32_t v, e;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(e) : "l"(p) : "memory");
  if (e != epoch) {
    const unsigned long long t0 = global_ns();
    do {
      if (global_ns() - t0 > timeout_ns) return false;
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(e) : "l"(p) : "memory");
    } while (e != epoch);
  }
  *out = __uint_as_float(v);
  return true;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// The same for two neighbouring entries (p 16-byte aligned) with one 16-byte load per poll.
__device__ __forceinline__ bool peer_ll_load2(const uint2* p, uint32_t epoch, unsigned long long timeout_ns, float* o0, float* o1) {
  uint32_t v0, e0, v1, e1;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(e0), "=r"(v1), "=r"(e1) : "l"(p) : "memory");
  if (e0 != epoch || e1 != epoch) {
    const unsigned long long t0 = global_ns();
    do {
      if (global_ns() - t0 > timeout_ns) return false;
      asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(e0), "=r"(v1), "=r"(e1) : "l"(p) : "memory");
    } while (e0 != epoch || e1 != epoch);
  }
  *o0 = __uint_as_float(v0);
  *o1 = __uint_as_float(v1);
  return true;
}


struct jg_comm;
// Fill the exchange-related fields of `a` (buffers, counters, rank, world, timeout) for this communicator and give the
// launch the next exchange number — or, with `consume`, the number of the exchange the preceding push started.
// JG_EINVAL when the peer buffers are not open.
int jg_peer_fill_args(jg_comm* comm, PeerArgs* a, bool consume = false);
