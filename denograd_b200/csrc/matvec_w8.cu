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
//   * a warp keeps U such loads in flight; the eight warps of a CTA take interleaved k blocks of the same 8-row tile
//     (512 contiguous bytes of every row per pass) and meet in shared memory once per tile, in a fixed order.
// Tiles are dealt to CTAs as contiguous runs, so the two CTAs of an SM finish within one tile of the others.
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

template <int EPI, bool NORM, int U>
__global__ void __launch_bounds__(W8_THREADS, 2) jg_matvec_w8_kernel(const MatvecW8Args a) {
  constexpr int NW = (EPI == W8_SWIGLU) ? 2 : 1;
  extern __shared__ __align__(16) unsigned char w8_smem[];  // [M rows][xstride] activations (rows >= M of the tile are zero registers)
  __shared__ float part[W8_WARPS][NW][2][32];               // per warp: the lane's two sums (c0, c1) of each matrix
  __shared__ float red[W8_WARPS];
  __shared__ float s_rs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, N = a.N, M = a.M;
  const int n_kb = K / 64;                                  // 64-wide k blocks
  const int n_tiles = (N + 7) / 8;
  const int tile0 = (int)((long long)blockIdx.x * n_tiles / gridDim.x);
  const int tile1 = (int)((long long)(blockIdx.x + 1) * n_tiles / gridDim.x);
  pdl_launch();

  // ---- weights of the first batch: they do not depend on the preceding kernel
  const int8_t* wsrc[NW];
  wsrc[0] = a.w0;
  if (NW == 2) wsrc[NW - 1] = a.w1;
  uint4 wv[NW][U];
  auto load_batch = [&](int tile, int kb0) {  // blocks kb0 + warp + 8u, u < U, of weight row tile*8 + g
    const int row = min(tile * 8 + g, N - 1);  // clamp: a duplicated row is never stored
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int kb = kb0 + warp + W8_WARPS * u;
#pragma unroll
      for (int w = 0; w < NW; w++)
        wv[w][u] = (kb < n_kb && tile < tile1) ? ld_stream_128(wsrc[w] + (size_t)row * K + (size_t)kb * 64 + t * 16) : make_uint4(0, 0, 0, 0);
    }
  };
  load_batch(tile0, 0);
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
  unsigned long long best0 = 0ull, best1 = 0ull;  // LOGITS: keys of the outputs this thread finishes (m = tid / 4 fixed)

  for (int tile = tile0; tile < tile1; tile++) {
    const int row = min(tile * 8 + g, N - 1);
    __half2 sc[NW];
    sc[0] = __half2half2(a.s0[row]);
    if (NW == 2) sc[NW - 1] = __half2half2(a.s1[row]);
    float acc[NW][4];
#pragma unroll
    for (int w = 0; w < NW; w++) acc[w][0] = acc[w][1] = acc[w][2] = acc[w][3] = 0.f;

    for (int kb0 = 0; kb0 < n_kb; kb0 += W8_WARPS * U) {
      // consume the batch in registers, then request the next one (the next tile's first batch at the end of a tile)
      uint4 cur[NW][U];
#pragma unroll
      for (int w = 0; w < NW; w++)
#pragma unroll
        for (int u = 0; u < U; u++) cur[w][u] = wv[w][u];
      if (kb0 + W8_WARPS * U < n_kb) load_batch(tile, kb0 + W8_WARPS * U);
      else load_batch(tile + 1, 0);
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int kb = kb0 + warp + W8_WARPS * u;
        if (kb < n_kb) {
          const uint4* xp = reinterpret_cast<const uint4*>(xrow + (size_t)kb * 128);
          const uint4 zero4 = make_uint4(0, 0, 0, 0);
          const uint4 x0 = has_row ? xp[0] : zero4, x1 = has_row ? xp[1] : zero4;
          const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
          for (int w = 0; w < NW; w++) {
            uint32_t d[8];
            w8_dequant16(cur[w][u], sc[w], d);
#pragma unroll
            for (int i = 0; i < 4; i++) w8_mma(acc[w], xw[2 * i], xw[2 * i + 1], d[2 * i], d[2 * i + 1]);
          }
        }
      }
    }
    // ---- the eight k slices meet in shared memory; warp 0 adds them in warp order and finishes the tile:
    //      lane (g, t) holds activation row g against weight rows tile*8 + 2t and + 2t + 1
#pragma unroll
    for (int w = 0; w < NW; w++) { part[warp][w][0][lane] = acc[w][0]; part[warp][w][1][lane] = acc[w][1]; }
    __syncthreads();
    if (warp == 0 && g < M) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int n = tile * 8 + 2 * t + e;
        if (n < N) {
          float s_a = 0.f, s_b = 0.f;
#pragma unroll
          for (int q = 0; q < W8_WARPS; q++) s_a += part[q][0][e][lane];
          if (NW == 2) {
#pragma unroll
            for (int q = 0; q < W8_WARPS; q++) s_b += part[q][NW - 1][e][lane];
          }
          const size_t o = (size_t)g * N + n;
          if (EPI == W8_PARTIAL) { a.y32[o] = s_a; continue; }
          __half v = __float2half_rn(s_a);
          if (EPI == W8_RESIDUAL) v = hadd1(a.residual[o], v);
          if (EPI == W8_SWIGLU) v = jg_silu_mul(v, __float2half_rn(s_b));
          a.y[o] = v;
          if (EPI == W8_LOGITS) {
            const unsigned long long k = argmax_key(v, (uint32_t)(n + a.row_offset));
            if (e == 0) best0 = k > best0 ? k : best0; else best1 = k > best1 ? k : best1;
          }
        }
      }
    }
    __syncthreads();  // `part` is rewritten by the next tile
  }

  if (EPI == W8_LOGITS && warp == 0) {
    // lanes with the same g finished outputs of activation row g: fold over t, one atomic per row
    unsigned long long b = best0 > best1 ? best0 : best1;
#pragma unroll
    for (int o = 1; o < 4; o <<= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
      b = other > b ? other : b;
    }
    if (t == 0 && g < M && b != 0ull) atomicMax(a.key + g, b);
  }
}

template <int EPI, bool NORM>
static int launch_w8(jg_dev* dev, const MatvecW8Args& a, const char* name) {
  constexpr int U = (EPI == W8_SWIGLU) ? 4 : 8;  // 16-byte loads in flight per lane and matrix
  auto kern = jg_matvec_w8_kernel<EPI, NORM, U>;
  const size_t smem = (size_t)a.M * a.xstride;
  static size_t smem_set[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  static int occ_for[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  static size_t occ_smem[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int slot = dev->ordinal & 7;
  if (smem > 40 * 1024 && smem > smem_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev->prop.sharedMemPerBlockOptin - 16 * 1024));
    smem_set[slot] = dev->prop.sharedMemPerBlockOptin;
  }
  if (occ_for[slot] == 0 || occ_smem[slot] != smem) {
    int occ = 0;
    JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, W8_THREADS, smem));
    occ_for[slot] = occ < 1 ? 1 : (occ > 2 ? 2 : occ);
    occ_smem[slot] = smem;
  }
  const int n_tiles = (a.N + 7) / 8;
  long long blocks = (long long)dev->sm_count * occ_for[slot];
  if (blocks > n_tiles) blocks = n_tiles;
  if (blocks < 1) blocks = 1;
  return jg_launch(dev, name, kern, dim3((unsigned)blocks), dim3(W8_THREADS), smem, a);
}

// Whether the shape is one this kernel takes: whole 64-wide k blocks, and M activation rows of K halves (plus padding)
// small enough for two CTAs per SM (with one CTA an SM has too few loads in flight to keep up with HBM).
bool jg_matvec_w8_fits(const jg_dev* dev, int M, int K) {
  return M >= 1 && M <= 8 && K % 64 == 0 && 2 * ((size_t)M * (2 * (size_t)K + 16) + 4 * 1024) <= (size_t)dev->prop.sharedMemPerMultiprocessor;
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
