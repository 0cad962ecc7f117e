// Dense projection on the 5th-generation tensor cores for 3 rows and more (batched decode, prompt processing):
// Y[m][n] = epilogue( sum_k X[m][k] * W[n][k] ) with tcgen05.mma, the accumulator in tensor memory and both operands
// brought into 128-byte swizzled shared memory by TMA (cp.async.bulk.tensor).
//
// The roles of the MMA are swapped with respect to the usual GEMM picture so that both operands are K-major exactly as
// they lie in memory (nn.Linear keeps W as [out][in], jsgrad/nn/index.ts:403-412): A = 128 weight rows x 64 k,
// B = TN activation rows x 64 k (TN = 16 ... 256), D[128 lanes = weight rows][TN columns = activation rows] in fp32.
// With few activation rows the kernel is a weight stream: every weight byte crosses HBM once, the pipeline is as deep
// as shared memory allows, and the first weight tiles are requested before the kernel waits for its predecessor.
// Warp roles: warp 0 issues the TMA loads (one lane), warp 1 owns tensor memory and issues the MMAs (one lane),
// warps 2-9 read the accumulator back (tcgen05.ld; a warp may touch the 32-lane quarter given by its id modulo 4, so
// two warps share a quarter and split its columns) and apply the epilogue.
//
// Split-K over a thread-block cluster: when the output tiles alone do not fill the GPU, the CTAs of a cluster
// (1,1,ks) share one output tile, each accumulating a slice of K; ranks > 0 then write their accumulators into rank 0's
// (by then idle) pipeline buffers through distributed shared memory and rank 0 adds them in rank order before the
// epilogue.  No cluster multicast is used anywhere: every CTA fetches its own tiles.
// int8 weights (Int8Linear with many rows, jsgrad/models/llama3.ts:35): the weight tile arrives by TMA as int8 (8 KB
// instead of 16), and the warps that will later run the epilogue — idle during the main loop — turn it into the fp16
// tile the MMA reads: thread = one weight row of the tile, half(q) * scale rounded once per element, written in the
// 128-byte swizzle pattern TMA would have produced (16-byte chunk c of row r lands at chunk c ^ (r % 8)), followed by a
// proxy fence.  The weights cross HBM as int8 once per pass; no fp16 copy of a matrix is ever written.
// Every mbarrier wait is bounded: a wait that does not complete sets an error word and the CTA winds down (cluster
// barriers are still reached, tensor memory is released in every case); the host reports JG_ETIMEDOUT at the next
// synchronisation.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "transcendental.cuh"

enum { TC_STORE = 0, TC_RESIDUAL = 1, TC_SWIGLU = 2, TC_PARTIAL = 4 };

constexpr int TC_BM = 128;  // weight rows per CTA (MMA M)
constexpr int TC_BK = 64;   // k per stage: 64 halves = one 128-byte swizzle row
// Threads of a CTA: warp 0 TMA, warp 1 MMA, then EPW epilogue warps for each 32-lane quarter of tensor memory.
constexpr int tc_threads(int epw) { return 64 + 128 * epw; }
// Polls of one mbarrier phase before a wait gives up.  A try_wait that fails returns after the hardware's own
// suspend time (up to ~1 us), so the limit is of the order of seconds; every wait starts after the kernel's dependency
// wait, i.e. it only ever measures this kernel's own TMA / MMA progress.
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

struct TcArgs {
  __half* y;
  float* y32;
  const __half* residual;
  int* err;  // device word: 0 = fine, otherwise the code of the first wait that gave up
  int M, N, K;
  int w_late;  // the weights were written by the preceding kernel: no load before the dependency wait
  const __half* s0;  // int8 weights: per-output-row scales of the (first / second) matrix
  const __half* s1;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}
// K-major operand tile in 128-byte swizzled shared memory: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
  const uint32_t lo = ((smem_u32(tile) & 0x3FFFFu) >> 4) | (1u << 16);  // start address, leading byte offset = 1 (unused)
  const uint32_t hi = 64u | (1u << 14) | (2u << 29);                    // stride 1024 B, descriptor version 1, SWIZZLE_128B
  return (uint64_t)lo | ((uint64_t)hi << 32);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&r)[16]) {
  uint32_t u[16];
  tmem_ld16(taddr, u);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 16; j++) r[j] = __uint_as_float(u[j]);
}
// Cluster-wide barrier with release / acquire semantics (orders the distributed-shared-memory traffic around it).
__device__ __forceinline__ void cluster_barrier() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Shared-memory address `local` as seen in the CTA of rank `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

template <int TN, int EPI, bool W8 = false, bool HALF = false>
struct TcCfg {
  static constexpr int NW = (EPI == TC_SWIGLU) ? 2 : 1;
  static constexpr uint32_t RAW_BYTES = W8 ? TC_BM * TC_BK : 0;  // the int8 tile as it arrives (8 KB)
  static constexpr int NCOL = NW * TN;                 // accumulator columns
  // epilogue warps per tensor-memory quarter: wide tiles leave each of them 64 columns (measured at 512 rows: 12.1 ->
  // 11.8 ms per prefill against two warps), narrow ones are over before more warps would pay (batch 32: 6.92k tok/s
  // with two, 6.84k with four)
  static constexpr int EPW = TN >= 128 ? 4 : 2;
  static constexpr int THREADS = tc_threads(EPW);
  static constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;  // 16 KB
  static constexpr uint32_t B_BYTES = TN * TC_BK * 2;
  static constexpr uint32_t STAGE_BYTES = NW * (A_BYTES + RAW_BYTES) + B_BYTES;  // [A0 | A1 | B | raw0 | raw1]
  // int8: every epilogue warp converts during the main loop, in CONV_SPLIT groups (EPW / NW: 1, 2 or 4) of four warps per
  // matrix (one thread per weight row); group g takes the k-blocks g, g + CONV_SPLIT, ..., so that many k-blocks are being
  // converted at once and a group's fixed costs (barrier wait, proxy fence, arrival) hide behind the other groups' work
  static constexpr int CONV_SPLIT = W8 ? (EPW / NW >= 1 ? EPW / NW : 1) : 1;
  static constexpr int CONV_WARPS = W8 ? 4 * NW * CONV_SPLIT : 0;
  // HALF: a ring of half the shared memory, so that two CTAs share an SM (few activation rows only)
  static constexpr int STAGES_FIT = ((HALF ? 110 : 225) * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 10 ? 10 : STAGES_FIT;
  static constexpr uint32_t TMEM_COLS = NCOL <= 32 ? 32 : (NCOL <= 64 ? 64 : (NCOL <= 128 ? 128 : (NCOL <= 256 ? 256 : 512)));
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
  // split-K peers park their accumulators ([column][128 lanes] fp32 each) in rank 0's pipeline buffers
  static constexpr int MAX_KS = 1 + (int)(((size_t)STAGES * STAGE_BYTES) / ((size_t)NCOL * TC_BM * 4));
};

// int8 x16 -> sixteen halves of half(q) * s (eight half2 registers in k order), each product rounded once
__device__ __forceinline__ void tc_dequant16(const uint4& raw, __half2 s2, uint32_t (&out)[8]) {
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);  // 1024 + 128
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t v = words[i] ^ 0x80808080u;          // signed -> offset-binary
    uint32_t lo = __byte_perm(v, 0x64646464u, 0x4140);  // bytes 0,1 -> halves 1024 + b
    uint32_t hi = __byte_perm(v, 0x64646464u, 0x4342);  // bytes 2,3
    const __half2 p = __hmul2_rn(__hsub2(*reinterpret_cast<__half2*>(&lo), bias), s2);
    const __half2 q = __hmul2_rn(__hsub2(*reinterpret_cast<__half2*>(&hi), bias), s2);
    out[2 * i] = *reinterpret_cast<const uint32_t*>(&p);
    out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&q);
  }
}

template <int TN, int EPI, bool W8 = false, bool HALF = false>
__global__ void __launch_bounds__(TcCfg<TN, EPI, W8, HALF>::THREADS, HALF ? 2 : 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w0,
                                                             const __grid_constant__ CUtensorMap tm_w1,
                                                             const __grid_constant__ CUtensorMap tm_x, const TcArgs a) {
  using Cfg = TcCfg<TN, EPI, W8, HALF>;
  constexpr int NW = Cfg::NW, STAGES = Cfg::STAGES, NCOL = Cfg::NCOL;
  constexpr uint32_t A_BYTES = Cfg::A_BYTES, STAGE_BYTES = Cfg::STAGE_BYTES, TMEM_COLS = Cfg::TMEM_COLS;
  constexpr uint32_t RAW_BYTES = Cfg::RAW_BYTES, B_BYTES = Cfg::B_BYTES, RAW_OFF = NW * A_BYTES + B_BYTES;
  static_assert(!W8 || Cfg::CONV_WARPS <= 4 * Cfg::EPW, "the converting warps are epilogue warps");
  __shared__ __align__(8) uint64_t raw_full[W8 ? STAGES : 1], a_full[W8 ? STAGES : 1];
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t s_tmem;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok0 = blockIdx.x * TN, feat0 = blockIdx.y * TC_BM;
  const int ks = gridDim.z, rank = blockIdx.z;  // the cluster is (1,1,ks): the rank in it is blockIdx.z
  const int n_kb = a.K / TC_BK;
  const int kb0 = (int)((long long)rank * n_kb / ks), nk = (int)((long long)(rank + 1) * n_kb / ks) - kb0;
  pdl_launch();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    if (W8)
      for (int s = 0; s < STAGES; s++) { mbar_init(&raw_full[s], 1); mbar_init(&a_full[s], 4 * NW); }
    mbar_init(&acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory for the accumulator(s): one warp allocates, the same warp frees
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem;
  bool acc_ok = false;

  if (warp == 0 && lane == 0) {
    // ---- producer.  Weights do not depend on the preceding kernel: the first tiles are requested before the wait.
    const int pre = nk < STAGES ? nk : STAGES;
    if (a.w_late) pdl_wait();
    // fp16 weights land in the A tiles and complete full_bar together with the activations; int8 weights land in the
    // raw tiles and complete raw_full (the converting warps then fill the A tiles and complete a_full)
    auto load_w = [&](int i, int s) {
      unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
      if (W8) {
        mbar_expect_tx(&raw_full[s], NW * RAW_BYTES);
        tma_load_2d(st + RAW_OFF, &tm_w0, (kb0 + i) * TC_BK, feat0, &raw_full[s]);
        if (NW == 2) tma_load_2d(st + RAW_OFF + RAW_BYTES, &tm_w1, (kb0 + i) * TC_BK, feat0, &raw_full[s]);
        mbar_expect_tx(&full_bar[s], B_BYTES);
      } else {
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(st, &tm_w0, (kb0 + i) * TC_BK, feat0, &full_bar[s]);
        if (NW == 2) tma_load_2d(st + A_BYTES, &tm_w1, (kb0 + i) * TC_BK, feat0, &full_bar[s]);
      }
    };
    for (int i = 0; i < pre; i++) load_w(i, i);
    pdl_wait();  // X comes from the previous kernel
    for (int i = 0; i < pre; i++)
      tma_load_2d(tiles + (size_t)i * STAGE_BYTES + NW * A_BYTES, &tm_x, (kb0 + i) * TC_BK, tok0, &full_bar[i]);
    for (int i = pre; i < nk; i++) {
      const int s = i % STAGES;
      // the MMAs of the stage's previous use are done: its A and B tiles are free, and so is its raw tile (converted
      // before those MMAs could start)
      if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) { atomicCAS(a.err, 0, 1); break; }
      load_w(i, s);
      tma_load_2d(tiles + (size_t)s * STAGE_BYTES + NW * A_BYTES, &tm_x, (kb0 + i) * TC_BK, tok0, &full_bar[s]);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer: 4 x (128 x TN x 16) per stage and matrix, accumulating in tensor memory
    const uint32_t idesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);  // f32 acc, f16 x f16, K-major both
    bool ok = true;
    // the poll budget of the waits below starts only once the predecessor is done: the producer cannot request the
    // activation tiles any earlier, so a slow predecessor must not use the budget up
    pdl_wait();
    for (int i = 0; i < nk; i++) {
      const int s = i % STAGES;
      if (!mbar_wait(&full_bar[s], (i / STAGES) & 1)) { atomicCAS(a.err, 0, 2); ok = false; break; }
      if (W8 && !mbar_wait(&a_full[s], (i / STAGES) & 1)) { atomicCAS(a.err, 0, 2); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
      const uint64_t bdesc = umma_desc(st + NW * A_BYTES);
#pragma unroll
      for (int w = 0; w < NW; w++) {
        const uint64_t adesc = umma_desc(st + w * A_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; k++)  // 16 halves = 32 bytes further along K inside the swizzle row: +2 (16-byte units)
          umma_f16(tmem_base + w * TN, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(&empty_bar[s]);  // arrives when the MMAs above have finished reading the stage
    }
    if (ok) umma_commit(&acc_bar);  // ... and when the whole accumulation is complete
  } else if (warp >= 2) {
    if (W8 && warp - 2 < Cfg::CONV_WARPS) {
      // ---- converter: this thread's weight row of every stage, int8 -> half(q) * scale -> swizzled fp16 tile
      constexpr int CS = Cfg::CONV_SPLIT;
      const int cw = warp - 2, w = cw / (4 * CS), idx = cw % (4 * CS), r = (idx & 3) * 32 + lane, group = idx >> 2;
      if (a.w_late) pdl_wait();
      const __half2 sc = __half2half2((w == 0 ? a.s0 : a.s1)[min(feat0 + r, a.N - 1)]);
      const uint32_t row_off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
      for (int i = group; i < nk; i += CS) {
        const int s = i % STAGES;
        if (!mbar_wait(&raw_full[s], (i / STAGES) & 1)) { atomicCAS(a.err, 0, 1); break; }
        unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
        const uint4* src = reinterpret_cast<const uint4*>(st + RAW_OFF + w * RAW_BYTES + r * TC_BK);
        unsigned char* dst = st + w * A_BYTES + row_off;
#pragma unroll
        for (int j = 0; j < 4; j++) {  // 16 weights -> two 16-byte chunks (2j, 2j + 1) of the row
          uint32_t d[8];
          tc_dequant16(src[j], sc, d);
          *reinterpret_cast<uint4*>(dst + (((2 * j) ^ (r & 7)) << 4)) = make_uint4(d[0], d[1], d[2], d[3]);
          *reinterpret_cast<uint4*>(dst + (((2 * j + 1) ^ (r & 7)) << 4)) = make_uint4(d[4], d[5], d[6], d[7]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the MMA's reads
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&a_full[s])) : "memory");
      }
    }
    pdl_wait();  // the residual is read and Y written only after the previous kernel is done with them
    acc_ok = mbar_wait(&acc_bar, 0);
    if (!acc_ok && lane == 0) atomicCAS(a.err, 0, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }

  // warp (id % 4) may touch tensor-memory lanes [32 * (id % 4), +32); lane l of it is weight row feat0 + 32q + l
  const int q = warp & 3, row = q * 32 + lane;
  // the two warps of a quarter split the accumulator columns (activation rows) between them
  const int part = (warp - 2) >> 2;
  constexpr int TN_PER = (TN / Cfg::EPW) >= 16 ? (TN / Cfg::EPW) : 16;
  constexpr int NC_PER = (NCOL / Cfg::EPW) >= 16 ? (NCOL / Cfg::EPW) : 16;
  const int tn_lo = part * TN_PER, tn_hi = min(TN, tn_lo + TN_PER);
  const int nc_lo = part * NC_PER, nc_hi = min(NCOL, nc_lo + NC_PER);
  const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
  float* red = reinterpret_cast<float*>(tiles);  // rank 0: [ks-1][NCOL][128] partial accumulators of the peers
  if (ks > 1) {
    cluster_barrier();  // rank 0's MMAs have consumed its pipeline buffers (its epilogue warps waited for them)
    if (rank > 0 && warp >= 2 && acc_ok) {
      const uint32_t dst0 = map_to_rank(smem_u32(red + ((size_t)(rank - 1) * NCOL) * TC_BM + row), 0);
#pragma unroll 1
      for (int c0 = nc_lo; c0 < nc_hi; c0 += 16) {
        float r0[16];
        tmem_ld16(t_lane + c0, r0);
#pragma unroll
        for (int j = 0; j < 16; j++) st_cluster_f32(dst0 + (uint32_t)((c0 + j) * TC_BM * 4), r0[j]);
      }
    }
    cluster_barrier();  // the peers' partial sums have landed in rank 0
  }
  if (rank == 0 && warp >= 2 && acc_ok) {
    const int feat = feat0 + row;
#pragma unroll 1
    for (int c0 = tn_lo; c0 < tn_hi; c0 += 16) {
      float r0[16], r1[16];
      tmem_ld16(t_lane + c0, r0);
      if (NW == 2) tmem_ld16(t_lane + TN + c0, r1);
      for (int p = 1; p < ks; p++) {  // rank order
        const float* pr = red + ((size_t)(p - 1) * NCOL) * TC_BM + row;
#pragma unroll
        for (int j = 0; j < 16; j++) {
          r0[j] = __fadd_rn(r0[j], pr[(size_t)(c0 + j) * TC_BM]);
          if (NW == 2) r1[j] = __fadd_rn(r1[j], pr[(size_t)(TN + c0 + j) * TC_BM]);
        }
      }
      if (feat < a.N) {
        __half res[16];
        if (EPI == TC_RESIDUAL) {  // all loads first: Y may alias the residual, which would serialise load / store pairs
#pragma unroll
          for (int j = 0; j < 16; j++)
            res[j] = (tok0 + c0 + j < a.M) ? a.residual[(size_t)(tok0 + c0 + j) * a.N + feat] : __float2half_rn(0.f);
        }
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int tok = tok0 + c0 + j;
          if (tok < a.M) {
            const size_t o = (size_t)tok * a.N + feat;
            if (EPI == TC_PARTIAL) { a.y32[o] = r0[j]; continue; }
            __half v = __float2half_rn(r0[j]);
            if (EPI == TC_RESIDUAL) v = hadd1(res[j], v);
            if (EPI == TC_SWIGLU) v = jg_silu_mul(v, __float2half_rn(r1[j]));
            a.y[o] = v;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ CTA pairs
// The same projection with tcgen05.mma.cta_group::2 for many activation rows: two CTAs of a cluster (2,1,1) hold two
// adjacent 128-row weight tiles and share one 256-row activation tile, each fetching only its half of it (rows
// 128 * rank ..): the MMAs, issued by rank 0 for both, read A from each CTA's own shared memory into that CTA's tensor
// memory and the two halves of B from both.  Per k-block a CTA moves 32 KB (48 KB for the gate / up pair) instead of 48 KB
// (64 KB) for the same MMA work, and the ring is 7 (4) stages deep instead of 4 (3).
// Signals: every TMA load of either CTA completes on rank 0's full barrier (cp.async.bulk.tensor with .cta_group::2 may
// name the peer's barrier; no multicast anywhere); the MMA issuer commits each stage to both CTAs' empty barriers and
// the final accumulation to both CTAs' accumulator barriers (one tcgen05.commit per CTA).  Tensor memory is allocated
// and released by warp 1 of both CTAs together (.cta_group::2).  No split-K.
template <int EPI>
struct Tc2Cfg {
  static constexpr int NW = (EPI == TC_SWIGLU) ? 2 : 1;
  static constexpr int TN = 256;                        // activation rows of the pair's tile
  static constexpr int NCOL = NW * TN;
  static constexpr int EPW = 4;
  static constexpr int THREADS = tc_threads(EPW);
  static constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;       // 16 KB: this CTA's weight rows
  static constexpr uint32_t B_BYTES = (TN / 2) * TC_BK * 2;    // 16 KB: this CTA's half of the activation tile
  static constexpr uint32_t STAGE_BYTES = NW * A_BYTES + B_BYTES;
  static constexpr int STAGES_FIT = (225 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 10 ? 10 : STAGES_FIT;
  static constexpr uint32_t TMEM_COLS = NCOL <= 256 ? 256 : 512;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
};

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at shared::cluster address `bar` once the pair's MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(Tc2Cfg<EPI>::THREADS) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_w0,
                                                                            const __grid_constant__ CUtensorMap tm_w1,
                                                                            const __grid_constant__ CUtensorMap tm_x, const TcArgs a) {
  using Cfg = Tc2Cfg<EPI>;
  constexpr int NW = Cfg::NW, STAGES = Cfg::STAGES, TN = Cfg::TN;
  constexpr uint32_t A_BYTES = Cfg::A_BYTES, STAGE_BYTES = Cfg::STAGE_BYTES, TMEM_COLS = Cfg::TMEM_COLS;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t s_tmem;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  // grid (2 x activation tiles, pairs of weight tiles): the two CTAs of a pair are neighbours along x (a launch whose
  // pairs lay along y was refused as a cluster misconfiguration), and the pairs that share weights follow each other
  const int tok0 = (int)(blockIdx.x >> 1) * TN, feat0 = ((int)blockIdx.y * 2 + (int)rank) * TC_BM;
  const int nk = a.K / TC_BK;
  pdl_launch();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // warp 1 of both CTAs together: the same columns of both CTAs' tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_barrier();  // the peer's barriers exist before anything is signalled across
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem;
  bool acc_ok = false;

  if (warp == 0 && lane == 0) {
    // ---- producer of this CTA's tiles; all completions go to rank 0's full barrier, which rank 0 arms for both CTAs
    const int pre = nk < STAGES ? nk : STAGES;
    if (a.w_late) pdl_wait();
    auto full0 = [&](int s) { return map_to_rank(smem_u32(&full_bar[s]), 0); };
    auto load_w = [&](int i, int s) {
      unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
      if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
      tma_load_2d_pair(st, &tm_w0, i * TC_BK, feat0, full0(s));
      if (NW == 2) tma_load_2d_pair(st + A_BYTES, &tm_w1, i * TC_BK, feat0, full0(s));
    };
    auto load_x = [&](int i, int s) {
      tma_load_2d_pair(tiles + (size_t)s * STAGE_BYTES + NW * A_BYTES, &tm_x, i * TC_BK, tok0 + (int)rank * (TN / 2), full0(s));
    };
    for (int i = 0; i < pre; i++) load_w(i, i);
    pdl_wait();  // X comes from the previous kernel
    for (int i = 0; i < pre; i++) load_x(i, i);
    for (int i = pre; i < nk; i++) {
      const int s = i % STAGES;
      if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) { atomicCAS(a.err, 0, 1); break; }
      load_w(i, s);
      load_x(i, s);
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issuer of the pair: 4 x (256 x 256 x 16) per stage and matrix
    const uint32_t idesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)((2 * TC_BM) >> 4) << 24);
    bool ok = true;
    pdl_wait();
    for (int i = 0; i < nk; i++) {
      const int s = i % STAGES;
      if (!mbar_wait(&full_bar[s], (i / STAGES) & 1)) { atomicCAS(a.err, 0, 2); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
      const uint64_t bdesc = umma_desc(st + NW * A_BYTES);
#pragma unroll
      for (int w = 0; w < NW; w++) {
        const uint64_t adesc = umma_desc(st + w * A_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; k++)
          umma_f16_pair(tmem_base + w * TN, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit_pair(smem_u32(&empty_bar[s]));                  // this CTA's stage is free ...
      umma_commit_pair(map_to_rank(smem_u32(&empty_bar[s]), 1));  // ... and the peer's
    }
    if (ok) {
      umma_commit_pair(smem_u32(&acc_bar));
      umma_commit_pair(map_to_rank(smem_u32(&acc_bar), 1));
    }
  } else if (warp >= 2) {
    pdl_wait();  // the residual is read and Y written only after the previous kernel is done with them
    acc_ok = mbar_wait(&acc_bar, 0);
    if (!acc_ok && lane == 0) atomicCAS(a.err, 0, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }

  // lane l of quarter q is weight row feat0 + 32q + l of this CTA; the four warps of a quarter split the columns
  const int q = warp & 3, row = q * 32 + lane;
  const int part = (warp - 2) >> 2;
  constexpr int TN_PER = TN / Cfg::EPW;
  const int tn_lo = part * TN_PER, tn_hi = tn_lo + TN_PER;
  const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
  if (warp >= 2 && acc_ok) {
    const int feat = feat0 + row;
#pragma unroll 1
    for (int c0 = tn_lo; c0 < tn_hi; c0 += 16) {
      float r0[16], r1[16];
      tmem_ld16(t_lane + c0, r0);
      if (NW == 2) tmem_ld16(t_lane + TN + c0, r1);
      if (feat < a.N) {
        __half res[16];
        if (EPI == TC_RESIDUAL) {
#pragma unroll
          for (int j = 0; j < 16; j++)
            res[j] = (tok0 + c0 + j < a.M) ? a.residual[(size_t)(tok0 + c0 + j) * a.N + feat] : __float2half_rn(0.f);
        }
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int tok = tok0 + c0 + j;
          if (tok < a.M) {
            const size_t o = (size_t)tok * a.N + feat;
            if (EPI == TC_PARTIAL) { a.y32[o] = r0[j]; continue; }
            __half v = __float2half_rn(r0[j]);
            if (EPI == TC_RESIDUAL) v = hadd1(res[j], v);
            if (EPI == TC_SWIGLU) v = jg_silu_mul(v, __float2half_rn(r1[j]));
            a.y[o] = v;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_barrier();  // neither CTA leaves, or gives its tensor memory back, while the other may still use either's
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static encode_tiled_fn g_encode = nullptr;

// `bytes` = element size: 2 for fp16 operands (128-byte swizzle, the layout the MMA descriptors name), 1 for int8
// weight tiles, which land unswizzled (64-byte rows) for the converting warps
static int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, const char* what, int bytes = 2) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || fn == nullptr) {
      jg_set_error("cuTensorMapEncodeTiled is not available from this driver");
      return JG_ENOTSUP;
    }
    g_encode = (encode_tiled_fn)fn;
  }
  const cuuint64_t dims[2] = {cols, rows};           // innermost first
  const cuuint64_t strides[1] = {cols * (cuuint64_t)bytes};  // bytes between rows
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        bytes == 2 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    jg_set_error("tensor map for %s (%llu x %llu) rejected: CUresult %d", what, (unsigned long long)rows, (unsigned long long)cols, (int)r);
    return JG_EINVAL;
  }
  return JG_OK;
}

// Encoded maps are kept per (base, rows, cols, box rows): a model's weights and workspaces keep their addresses, so a
// step after the first finds all of its maps here instead of encoding three per launch.
struct MapKey { const void* base; uint64_t rows, cols; uint32_t box_rows; int bytes; };
struct MapSlot { MapKey k; CUtensorMap m; bool used; };
constexpr int MAP_SLOTS = 1024;
static MapSlot g_maps[MAP_SLOTS];

static int cached_map(const CUtensorMap** out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, const char* what, int bytes = 2) {
  uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull ^ (rows * 0xBF58476D1CE4E5B9ull) ^ (cols << 20) ^ box_rows ^ ((uint64_t)bytes << 40);
  h ^= h >> 29;
  for (int probe = 0; probe < 8; probe++) {
    MapSlot& s = g_maps[(h + probe) % MAP_SLOTS];
    if (s.used && s.k.base == base && s.k.rows == rows && s.k.cols == cols && s.k.box_rows == box_rows && s.k.bytes == bytes) { *out = &s.m; return JG_OK; }
    if (!s.used) {
      int rc = make_map(&s.m, base, rows, cols, box_rows, what, bytes);
      if (rc) return rc;
      s.k = MapKey{base, rows, cols, box_rows, bytes};
      s.used = true;
      *out = &s.m;
      return JG_OK;
    }
  }
  MapSlot& s = g_maps[h % MAP_SLOTS];  // neighbourhood full: replace
  int rc = make_map(&s.m, base, rows, cols, box_rows, what, bytes);
  if (rc) { s.used = false; return rc; }
  s.k = MapKey{base, rows, cols, box_rows, bytes};
  s.used = true;
  *out = &s.m;
  return JG_OK;
}

template <int TN, int EPI, bool W8 = false, bool HALF = false>
static int launch_tc(jg_dev* dev, const void* x, const void* w0, const void* w1, TcArgs a) {
  using Cfg = TcCfg<TN, EPI, W8, HALF>;
  auto kern = gemm_tc_kernel<TN, EPI, W8, HALF>;
  static bool attr_set[8] = {false, false, false, false, false, false, false, false};
  const int slot = dev->ordinal & 7;
  if (!attr_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
    attr_set[slot] = true;
  }
  const CUtensorMap *pw0, *pw1, *px;
  int rc = cached_map(&pw0, w0, a.N, a.K, TC_BM, "weights", W8 ? 1 : 2);
  if (rc) return rc;
  rc = cached_map(&pw1, Cfg::NW == 2 ? w1 : w0, a.N, a.K, TC_BM, "weights (second matrix)", W8 ? 1 : 2);
  if (rc) return rc;
  rc = cached_map(&px, x, a.M, a.K, TN, "activations");
  if (rc) return rc;
  const CUtensorMap tw0 = *pw0, tw1 = *pw1, tx = *px;
  // up to 128 rows (weight streaming): split K over a cluster until the launch has CTAs for about two thirds of the
  // SMs, keeping at least 8 k-blocks per CTA and the peers' partial sums within rank 0's pipeline buffers
  const int tiles = ((a.M + TN - 1) / TN) * (a.N / TC_BM), n_kb = a.K / TC_BK;
  static int ks_env = -1;
  if (ks_env < 0) { const char* e = getenv("JG_TC_SPLITK"); ks_env = e ? atoi(e) : 0; }
  int ks = 1;
  if (a.M > 128) {
    // compute-bound tiles: the launch runs in waves of one CTA per SM, each costing its k-blocks (0.28 us apiece at
    // the tensor peak) plus about 18 us of fill, epilogue and cluster reduction (measured cold at 512 and 1024 rows:
    // qkv 36.9 us unsplit against 53.3 split in two, which makes 192 CTAs = two waves; wo 38.9 against 34.8; the
    // down projection 96.3 against 69.7).  Take the split with the smallest estimate.
    float best = 0.f;
    for (int c = 1; c <= Cfg::MAX_KS && c <= 8 && n_kb / c >= 8; c++) {
      const int waves = (tiles * c + dev->sm_count - 1) / dev->sm_count;
      const float t = (float)waves * ((float)(n_kb / c) * 0.28f + 18.f);
      if (c == 1 || t < best) { best = t; ks = c; }
    }
  } else {
    // half-size rings (two CTAs per SM): CTAs for four thirds of the SMs, but no more than four to a tile — beyond
    // that the cluster reduction costs more than the shorter streams save (wo at 32 rows: 18.5 us split in 4, 20.5 in 7)
    while (ks < (HALF ? 4 : 8) && ks < Cfg::MAX_KS && tiles * ks * 3 < dev->sm_count * 2 * (HALF ? 2 : 1) && n_kb / (ks + 1) >= 8) ks++;
  }
  if (ks_env >= 1 && ks_env <= 8 && ks_env <= Cfg::MAX_KS && n_kb / ks_env >= 1) ks = ks_env;
  dev->tc_pending = true;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.M + TN - 1) / TN, a.N / TC_BM, ks);  // activation tiles fastest: CTAs sharing weights run together
  cfg.blockDim = dim3(Cfg::THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (ks > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = ks;
    na++;
  }
  if (dev->pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw0, tw1, tx, a);
  if (e != cudaSuccess) return jg_cuda_fail(e, "gemm_tc", __FILE__, __LINE__);
  return jg_after_launch(dev, "gemm_tc");
}

// CTA pairs (gemm_tc_pair_kernel): fp16 weights, more than 128 rows, an even number of weight tiles.  Used for the
// gate / up pair, the one projection that cannot split K and that the pairs serve 2-7 % faster at every row count
// measured (8B shapes, us per launch, pairs against single CTAs: 256 rows 80 / 86, 512 rows 131 / 139, 768 rows 188 /
// 191, 1536 rows 307 / 311, 2048 rows 427 / 423); the single-matrix projections are level or slower in pairs (they lose
// their split-K at few rows: down projection at 512 rows 90 against 70 us), so they take them only when forced
// (JG_TC_PAIR=2; JG_TC_PAIR=0 turns the pairs off).
template <int EPI>
static int launch_tc_pair(jg_dev* dev, const void* x, const void* w0, const void* w1, TcArgs a) {
  using Cfg = Tc2Cfg<EPI>;
  auto kern = gemm_tc_pair_kernel<EPI>;
  static bool attr_set[8] = {false, false, false, false, false, false, false, false};
  const int slot = dev->ordinal & 7;
  if (!attr_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
    attr_set[slot] = true;
  }
  const CUtensorMap *pw0, *pw1, *px;
  int rc = cached_map(&pw0, w0, a.N, a.K, TC_BM, "weights");
  if (rc) return rc;
  rc = cached_map(&pw1, Cfg::NW == 2 ? w1 : w0, a.N, a.K, TC_BM, "weights (second matrix)");
  if (rc) return rc;
  rc = cached_map(&px, x, a.M, a.K, Cfg::TN / 2, "activations (half tile)");
  if (rc) return rc;
  const CUtensorMap tw0 = *pw0, tw1 = *pw1, tx = *px;
  dev->tc_pending = true;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ((a.M + Cfg::TN - 1) / Cfg::TN), a.N / (2 * TC_BM), 1);
  cfg.blockDim = dim3(Cfg::THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = 2;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = 1;
  na++;
  if (dev->pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw0, tw1, tx, a);
  if (e != cudaSuccess) return jg_cuda_fail(e, "gemm_tc_pair", __FILE__, __LINE__);
  return jg_after_launch(dev, "gemm_tc_pair");
}

static bool tc_pair_wanted(const TcArgs& a, bool gate_up) {
  static int env = -1;
  if (env < 0) { const char* e = getenv("JG_TC_PAIR"); env = e ? atoi(e) : 1; }
  if (env == 0 || a.s0 != nullptr || a.M <= 128 || (a.N / TC_BM) % 2 != 0) return false;
  return env == 2 || gate_up;
}

template <int EPI>
static int launch_tc_rows(jg_dev* dev, const void* x, const void* w0, const void* w1, const TcArgs& a) {
  if (tc_pair_wanted(a, EPI == TC_SWIGLU)) return launch_tc_pair<EPI>(dev, x, w0, w1, a);
  if (a.s0 != nullptr) {  // int8 weights: used from 20 rows on (fewer go to the mma.sync kernel)
    if (a.M <= 32) return launch_tc<32, EPI, true>(dev, x, w0, w1, a);
    if (a.M <= 128) return launch_tc<128, EPI, true>(dev, x, w0, w1, a);
    return launch_tc<256, EPI, true>(dev, x, w0, w1, a);
  }
  // Up to 32 rows the single-matrix projections run with half-size rings, two CTAs to an SM and twice the split-K:
  // a qkv or wo launch is a few hundred KB per CTA, mostly fixed cost (measured cold and alone at 32 rows on the 8B
  // shapes: qkv 29.2 -> 22.6 us, wo 19.4 -> 18.5 at split 4, down 36.9 -> 37.9; the batch-32 decode step 4.27 -> 4.16 ms,
  // batch 16 4.04 -> 3.93).  JG_TC_HALF=0 turns it off.  The gate / up pair keeps the full ring (three stages would
  // not cover its loads).
  static int half_env = -1;
  if (half_env < 0) { const char* e = getenv("JG_TC_HALF"); half_env = e ? atoi(e) : 1; }
  if (half_env && EPI != TC_SWIGLU && a.M <= 32) {
    if (a.M <= 16) return launch_tc<16, EPI, false, true>(dev, x, w0, w1, a);
    return launch_tc<32, EPI, false, true>(dev, x, w0, w1, a);
  }
  if (a.M <= 16) return launch_tc<16, EPI>(dev, x, w0, w1, a);
  if (a.M <= 32) return launch_tc<32, EPI>(dev, x, w0, w1, a);
  if (a.M <= 64) return launch_tc<64, EPI>(dev, x, w0, w1, a);
  if (a.M <= 128) return launch_tc<128, EPI>(dev, x, w0, w1, a);
  return launch_tc<256, EPI>(dev, x, w0, w1, a);
}

// Whether jg_gemm_tc takes this shape: fp16 weights, whole 128-row weight tiles and 64-wide k-blocks.
bool jg_gemm_tc_fits(int N, int K) { return N % TC_BM == 0 && K % TC_BK == 0; }

// Entry used by gemv.cu's public functions (fp16 weights, N % 128 == 0, K % 64 == 0).
// s0 / s1: per-row scales of int8 weights (w0 / w1 then hold int8), or null for fp16 weights.
int jg_gemm_tc(jg_dev* dev, int epi, const void* x, const void* w0, const void* w1, void* y, const void* residual, int M, int N, int K,
               const void* s0, const void* s1) {
  if (!jg_gemm_tc_fits(N, K)) {
    jg_set_error("projection: M=%d rows need N %% 128 == 0 and K %% 64 == 0 (N=%d, K=%d); split the rows into chunks of 64", M, N, K);
    return JG_ENOTSUP;
  }
  JG_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w0 % 16) == 0, "projection: operands must be 16-byte aligned for TMA");
  if (dev->err_word == nullptr) {
    JG_REQUIRE(!dev->capturing, "first tensor-core projection on a device must not be inside a graph capture");
    JG_CUDA(cudaMalloc(&dev->err_word, sizeof(int)));
    JG_CUDA(cudaMemsetAsync(dev->err_word, 0, sizeof(int), dev->stream));
  }
  TcArgs a = {};
  a.y = (__half*)y; a.y32 = (float*)y; a.residual = (const __half*)residual; a.err = dev->err_word; a.M = M; a.N = N; a.K = K;
  a.w_late = jg_is_fresh(dev, w0) || jg_is_fresh(dev, w1) || jg_is_fresh(dev, s0) || jg_is_fresh(dev, s1);
  a.s0 = (const __half*)s0; a.s1 = (const __half*)(s1 ? s1 : s0);
  switch (epi) {
    case TC_STORE: return launch_tc_rows<TC_STORE>(dev, x, w0, w1, a);
    case TC_RESIDUAL: return launch_tc_rows<TC_RESIDUAL>(dev, x, w0, w1, a);
    case TC_SWIGLU: return launch_tc_rows<TC_SWIGLU>(dev, x, w0, w1, a);
    case TC_PARTIAL: return launch_tc_rows<TC_PARTIAL>(dev, x, w0, w1, a);
  }
  jg_set_error("projection: epilogue %d has no tensor-core variant for M=%d rows", epi, M);
  return JG_ENOTSUP;
}
