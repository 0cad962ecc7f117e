// Weight-streaming projection over int8 weights for up to 8 activation rows (Int8Linear, jsgrad/models/llama3.ts:27-35:
// y[m][n] = half( sum_k float( x[m][k] * half(half(q[n][k]) * s[n]) ) ), fp32 accumulation).
//
// The CUDA-core kernel (gemv.cu) spends ~80 instructions per 16 weight bytes on dequantise-widen-FMA and reaches half the
// HBM rate; the k-tiled tensor-core kernel (gemm_small.cu) keeps too few bytes in flight (a barrier per 512-wide k tile,
// one tile of look-ahead).  This kernel takes from each what works:
//   * the activation rows live in shared memory for the whole launch (normalised in the prologue when the caller passes
//     the RMSNorm weight: jsgrad/nn/index.ts:586-588), so the k loop has no barrier at all;
//   * the products run on the tensor cores (mma.sync.m16n8k16) with the roles swapped: the A operand is the activation
//     tile (rows >= M are zero), the B operand is 8 weight rows.  A lane's single 16-byte load — 16 int8 weights of row
//     g at k-offset 16t inside a 64-wide k block — is, after the exact half(q) * s dequantisation, the B fragment of
//     four instructions, because the k positions inside a block may be permuted as long as the activation fragment
//     (32 bytes of row g at the same offset) uses the same permutation;
//   * a warp keeps U loads of 16 bytes in flight per lane and refills each register as it is consumed.  Where a matrix has 8-row tiles enough to give every warp of the launch its
//     own (gate/up, the output layer), warps stream whole tiles independently — no barrier at all; smaller matrices
//     split K over groups of 2, 4 or 8 warps (interleaved k blocks: KS x 64 contiguous bytes of every row per pass)
//     that meet at a barrier of their own once per tile and add their sums in a fixed order.
// Tiles are dealt to the warp groups as contiguous runs.
// Epilogues: STORE, RESIDUAL, SWIGLU (two matrices), LOGITS (+ greedy key), PARTIAL (fp32), as in gemv.cu.
#include "common.cuh"
#include "transcendental.cuh"

enum { W8_STORE = 0, W8_RESIDUAL = 1, W8_SWIGLU = 2, W8_LOGITS = 3, W8_PARTIAL = 4 };

struct MatvecW8Args {
  const __half* x;       // [M][K]
  const __half* norm_w;  // [K] or null
  const int8_t* w0;      // [N][K]
  const int8_t* w1;      // SWIGLU: up projection
  const __half* s0;      // [N]
  const __half* s1;
  __half* y;             // [M][N]
  const __half* residual;
  unsigned long long* key;
  float* y32;
  int row_offset;
  float eps, recip_k;
  int M, N, K;
  int xstride;           // bytes between activation rows in shared memory: 2K + 16
};

constexpr int W8_THREADS = 256;
constexpr int W8_WARPS = 8;

__device__ __forceinline__ void w8_dequant16(const uint4& raw, __half2 s2, uint32_t (&out)[8]) {
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);  // 1024 + 128
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t v = words[i] ^ 0x80808080u;                  // signed -> offset-binary
    uint32_t lo = __byte_perm(v, 0x64646464u, 0x4140);          // bytes 0,1 -> halves 1024 + b
    uint32_t hi = __byte_perm(v, 0x64646464u, 0x4342);          // bytes 2,3
    const __half2 a = __hmul2_rn(__hsub2(*reinterpret_cast<__half2*>(&lo), bias), s2);  // exact integer, one rounding
    const __half2 b = __hmul2_rn(__hsub2(*reinterpret_cast<__half2*>(&hi), bias), s2);
    out[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
    out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
  }
}

__device__ __forceinline__ void w8_mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // rows 8..15 of the activation tile are zero (a1 = a3 = 0)
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

template <int EPI, bool NORM, int U, int KS>
__global__ void __launch_bounds__(W8_THREADS, 2) jg_matvec_w8_kernel(const MatvecW8Args a) {
  constexpr int NW = (EPI == W8_SWIGLU) ? 2 : 1;
  constexpr int GROUPS = W8_WARPS / KS;  // warp groups of a CTA, each on its own tile
  extern __shared__ __align__(16) unsigned char w8_smem[];  // [M rows][xstride] activations (rows >= M of the tile are zero registers)
  __shared__ float part[2][W8_WARPS][NW][2][32];            // per tile parity and warp: the lane's two sums (c0, c1) of each matrix
  __shared__ float red[W8_WARPS];
  __shared__ float s_rs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, N = a.N, M = a.M;
  const int n_kb = K / 64;                                  // 64-wide k blocks
  const int n_tiles = (N + 7) / 8;
  const int group = warp / KS, sub = warp % KS;             // this warp's group in the CTA and its k slice in the group
  const long long gg = (long long)blockIdx.x * GROUPS + group, n_groups = (long long)gridDim.x * GROUPS;
  const int tile0 = (int)(gg * n_tiles / n_groups);
  const int tile1 = (int)((gg + 1) * n_tiles / n_groups);
  pdl_launch();

  // ---- the weight stream.  U loads of 16 bytes per matrix stay in flight per lane: register u holds block
  //      (kb0 + sub + KS * u) of the current batch and is refilled with the block one batch further on (the next
  //      tile's at the end of a tile) the moment it has been consumed.  The host only launches this kernel when K / 64
  //      is a multiple of KS * U.  Weights do not depend on the preceding kernel: the first batch is requested before
  //      the dependency wait.  (A ring of k blocks in shared memory filled by cp.async — twice the bytes in flight —
  //      measured slower: 37.7 against 28.6 us for the 8B gate/up pair.)
  const int8_t* wsrc[NW];
  wsrc[0] = a.w0;
  if (NW == 2) wsrc[NW - 1] = a.w1;
  uint4 wv[NW][U];
  __half sc_next[NW];  // the row's scales travel a tile ahead
  auto load_block = [&](int tile, int kb, int u) {
    const int row = min(tile * 8 + g, N - 1);  // clamp: a duplicated row is never stored
#pragma unroll
    for (int w = 0; w < NW; w++)
      wv[w][u] = (tile < tile1) ? ld_stream_128(wsrc[w] + (size_t)row * K + (size_t)kb * 64 + t * 16) : make_uint4(0, 0, 0, 0);
  };
  auto load_scales = [&](int tile) {
    const int row = min(min(tile, max(tile1 - 1, tile0)) * 8 + g, N - 1);
    sc_next[0] = a.s0[row];
    if (NW == 2) sc_next[NW - 1] = a.s1[row];
  };
#pragma unroll
  for (int u = 0; u < U; u++) load_block(tile0, sub + KS * u, u);
  load_scales(tile0);
  pdl_wait();

  // ---- prologue: activation rows -> shared memory (normalised when NORM)
  for (int m = 0; m < M; m++) {
    unsigned char* xm = w8_smem + (size_t)m * a.xstride;
    const __half* xg = a.x + (size_t)m * K;
    if (NORM) {
      float ss = 0.f;
      for (int c = tid; c < K / 8; c += W8_THREADS) {
        float v[8];
        unpack8(ld_128(xg + (size_t)c * 8), v);
#pragma unroll
        for (int k = 0; k < 8; k++) ss = fmaf(v[k], v[k], ss);
      }
      ss = warp_sum(ss);
      __syncthreads();  // red / s_rs reuse across rows
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      if (tid == 0) {
        float tt = 0.f;
        for (int i = 0; i < W8_WARPS; i++) tt += red[i];
        s_rs = sqrtf(__fdiv_rn(1.0f, __fadd_rn(__fmul_rn(tt, a.recip_k), a.eps)));
      }
      __syncthreads();
      const float rs = s_rs;
      for (int c = tid; c < K / 8; c += W8_THREADS) {
        float v[8];
        unpack8(ld_128(xg + (size_t)c * 8), v);
        uint4 gv = ld_128(a.norm_w + (size_t)c * 8);
        const __half* gh = reinterpret_cast<const __half*>(&gv);
        __align__(16) __half o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = hmul1(__float2half_rn(__fmul_rn(v[k], rs)), gh[k]);
        reinterpret_cast<uint4*>(xm)[c] = *reinterpret_cast<uint4*>(o);
      }
    } else {
      for (int c = tid; c < K / 8; c += W8_THREADS) reinterpret_cast<uint4*>(xm)[c] = ld_128(xg + (size_t)c * 8);
    }
  }
  __syncthreads();

  const unsigned char* xrow = w8_smem + (size_t)min(g, M - 1) * a.xstride + t * 32;  // this lane's activation row
  const bool has_row = g < M;                                                        // rows >= M of the tile are zero
  unsigned long long best0 = 0ull;  // LOGITS: best key among the outputs this thread finishes (all of activation row g)

  // Outputs of one finished tile: the k slices of the group are added in warp order; lane (g, t) of the finishing
  // warp holds activation row g against weight rows tile*8 + 2t and + 2t + 1.
  auto finish_tile = [&](int tile) {
    const int buf = (tile - tile0) & 1;
    if (g < M) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int n = tile * 8 + 2 * t + e;
        if (n < N) {
          float s_a = 0.f, s_b = 0.f;
#pragma unroll
          for (int q = 0; q < KS; q++) s_a += part[buf][group * KS + q][0][e][lane];
          if (NW == 2) {
#pragma unroll
            for (int q = 0; q < KS; q++) s_b += part[buf][group * KS + q][NW - 1][e][lane];
          }
          const size_t o = (size_t)g * N + n;
          if (EPI == W8_PARTIAL) { a.y32[o] = s_a; continue; }
          __half v = __float2half_rn(s_a);
          if (EPI == W8_RESIDUAL) v = hadd1(a.residual[o], v);
          if (EPI == W8_SWIGLU) v = jg_silu_mul(v, __float2half_rn(s_b));
          a.y[o] = v;
          if (EPI == W8_LOGITS) {
            const unsigned long long k = argmax_key(v, (uint32_t)(n + a.row_offset));
            best0 = k > best0 ? k : best0;
          }
        }
      }
    }
  };

  for (int tile = tile0; tile < tile1; tile++) {
    __half2 sc[NW];
    sc[0] = __half2half2(sc_next[0]);
    if (NW == 2) sc[NW - 1] = __half2half2(sc_next[NW - 1]);
    load_scales(tile + 1);  // a tile ahead
    // two accumulator sets per matrix, used alternately: consecutive instructions do not wait for each other's result
    float acc[NW][2][4];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
      for (int j = 0; j < 2; j++) acc[w][j][0] = acc[w][j][1] = acc[w][j][2] = acc[w][j][3] = 0.f;

    for (int kb0 = 0; kb0 < n_kb; kb0 += KS * U) {
      const bool last = kb0 + KS * U >= n_kb;  // the refills of this batch belong to the next tile
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int kb = kb0 + sub + KS * u;
        uint4 cur[NW];
#pragma unroll
        for (int w = 0; w < NW; w++) cur[w] = wv[w][u];
        if (last) load_block(tile + 1, sub + KS * u, u);
        else load_block(tile, kb + KS * U, u);
        const uint4* xp = reinterpret_cast<const uint4*>(xrow + (size_t)kb * 128);
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        const uint4 x0 = has_row ? xp[0] : zero4, x1 = has_row ? xp[1] : zero4;
        const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int w = 0; w < NW; w++) {
          uint32_t d[8];
          w8_dequant16(cur[w], sc[w], d);
#pragma unroll
          for (int q = 0; q < 4; q++) w8_mma(acc[w][q & 1], xw[2 * q], xw[2 * q + 1], d[2 * q], d[2 * q + 1]);
        }
      }
    }
    // ---- the k slices of the group meet in shared memory at a barrier of the group's own, once per tile.  The sums
    //      are then finished by one warp of the group (taking turns) while the others go on with the next tile;
    //      `part` alternates between two copies, and the copy of tile i is only rewritten after the barrier of tile
    //      i+1, which the finishing warp reaches after it is done with tile i.  A group of one warp needs none of it.
    const int buf = (tile - tile0) & 1;
#pragma unroll
    for (int w = 0; w < NW; w++) {
      part[buf][warp][w][0][lane] = __fadd_rn(acc[w][0][0], acc[w][1][0]);
      part[buf][warp][w][1][lane] = __fadd_rn(acc[w][0][1], acc[w][1][1]);
    }
    if (KS == W8_WARPS) __syncthreads();
    else if (KS > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(KS * 32) : "memory");
    else __syncwarp();
    if (sub == ((tile - tile0) % KS)) finish_tile(tile);
  }
  if (EPI == W8_LOGITS) {
    // lanes with the same g finished outputs of activation row g: fold over t, one atomic per row and warp
    unsigned long long b = best0;
#pragma unroll
    for (int o = 1; o < 4; o <<= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
      b = other > b ? other : b;
    }
    if (t == 0 && g < M && b != 0ull) atomicMax(a.key + g, b);
  }
}

template <int EPI, bool NORM, int KS>
static int launch_w8_ks(jg_dev* dev, const MatvecW8Args& a, const char* name) {
  constexpr int U = (EPI == W8_SWIGLU) ? 4 : 8;  // 16-byte loads in flight per lane and matrix
  auto kern = jg_matvec_w8_kernel<EPI, NORM, U, KS>;
  const size_t smem = (size_t)a.M * a.xstride;
  static size_t smem_set[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  static int occ_for[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  static size_t occ_smem[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int slot = dev->ordinal & 7;
  if (smem > 32 * 1024 && smem > smem_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev->prop.sharedMemPerBlockOptin - 16 * 1024));
    smem_set[slot] = dev->prop.sharedMemPerBlockOptin;
  }
  if (occ_for[slot] == 0 || occ_smem[slot] != smem) {
    int occ = 0;
    JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, W8_THREADS, smem));
    occ_for[slot] = occ < 1 ? 1 : (occ > 2 ? 2 : occ);
    occ_smem[slot] = smem;
  }
  const long long n_tiles = (a.N + 7) / 8;
  const long long groups = W8_WARPS / KS;
  long long blocks = (long long)dev->sm_count * occ_for[slot];
  if (blocks * groups > n_tiles) blocks = (n_tiles + groups - 1) / groups;
  if (blocks < 1) blocks = 1;
  return jg_launch(dev, name, kern, dim3((unsigned)blocks), dim3(W8_THREADS), smem, a);
}

// K is split over as few warps as still gives (nearly) every warp of a full launch a tile of its own: a tile streamed by
// one warp needs no barrier, but a launch wants its loads spread over all SMs.
template <int EPI, bool NORM>
static int launch_w8(jg_dev* dev, const MatvecW8Args& a, const char* name) {
  const long long n_tiles = (a.N + 7) / 8, warps = (long long)dev->sm_count * 2 * W8_WARPS;
  static int forced = -1;
  if (forced < 0) { const char* e = getenv("JG_W8_KS"); forced = e ? atoi(e) : 0; }
  int ks = 8;
  if (n_tiles * 10 >= warps * 6) ks = 1;
  else if (n_tiles * 2 * 10 >= warps * 6) ks = 2;
  else if (n_tiles * 4 * 10 >= warps * 6) ks = 4;
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) ks = forced;
  constexpr int U = (EPI == W8_SWIGLU) ? 4 : 8;
  while (ks > 1 && (a.K / 64) % (ks * U) != 0) ks >>= 1;  // whole batches per tile (jg_matvec_w8_fits checked ks = 1)
  switch (ks) {
    case 1: return launch_w8_ks<EPI, NORM, 1>(dev, a, name);
    case 2: return launch_w8_ks<EPI, NORM, 2>(dev, a, name);
    case 4: return launch_w8_ks<EPI, NORM, 4>(dev, a, name);
  }
  return launch_w8_ks<EPI, NORM, 8>(dev, a, name);
}

// Whether the shape is one this kernel takes: whole 64-wide k blocks, and M activation rows of K halves (plus padding)
// small enough for two CTAs per SM (with one CTA an SM has too few loads in flight to keep up with HBM).
bool jg_matvec_w8_fits(const jg_dev* dev, int M, int K) {
  static int max_m = -1;  // one row by default: from 2 rows on the k-tiled kernel is ahead (8B shapes, batch 2: 571 against 545 tok/s)
  if (max_m < 0) { const char* e = getenv("JG_W8_RESIDENT_MAX_M"); max_m = e ? atoi(e) : 1; }
  return M >= 1 && M <= max_m && M <= 8 && K % 512 == 0 &&  // K / 64 a multiple of the 8 loads a lane keeps in flight
         2 * ((size_t)M * (2 * (size_t)K + 16) + 4 * 1024) <= (size_t)dev->prop.sharedMemPerMultiprocessor;
}

// Entry used by gemv.cu's public functions: int8 weights, M <= 8.  norm_w non-null fuses RMSNorm over K into the prologue.
int jg_matvec_w8(jg_dev* dev, int epi, const void* x, const void* norm_w, float eps, const void* w0, const void* w1,
                 const void* s0, const void* s1, void* y, const void* residual, void* key, int M, int N, int K, int row_offset) {
  MatvecW8Args a = {};
  a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.w0 = (const int8_t*)w0; a.w1 = (const int8_t*)w1;
  a.s0 = (const __half*)s0; a.s1 = (const __half*)s1; a.y = (__half*)y; a.residual = (const __half*)residual;
  a.key = (unsigned long long*)key; a.y32 = (float*)y; a.row_offset = row_offset; a.eps = eps;
  a.recip_k = (float)(1.0 / (double)K); a.M = M; a.N = N; a.K = K; a.xstride = 2 * K + 16;
  const bool norm = norm_w != nullptr;
#define JG_W8_CASE(E, NAME) case E: return norm ? launch_w8<E, true>(dev, a, NAME) : launch_w8<E, false>(dev, a, NAME);
  switch (epi) {
    JG_W8_CASE(W8_STORE, "linear")
    JG_W8_CASE(W8_RESIDUAL, "linear")
    JG_W8_CASE(W8_SWIGLU, "norm_swiglu")
    JG_W8_CASE(W8_LOGITS, "norm_logits_argmax")
    JG_W8_CASE(W8_PARTIAL, "linear_partial")
  }
#undef JG_W8_CASE
  jg_set_error("projection: unknown epilogue %d", epi);
  return JG_EINVAL;
}
