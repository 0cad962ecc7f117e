// Weight-streaming projection for up to 64 activation rows (batched decode, short prefill chunks) — int8 weights, fp16
// shapes off the tcgen05 tile grid, and the logits with their argmax keys:
//   y[m][n] = epilogue( sum_k x[m][k] * W[n][k] ),  fp16 operands, fp32 accumulation on the tensor cores.
//
// At these row counts the projection is still bound by reading W once from HBM, but the multiply-accumulate work no
// longer fits the CUDA cores, so the products run through mma.sync.m16n8k16 (16 weight rows x 8 activation rows per
// instruction).  Nothing is staged or shuffled for the weights: a lane's 16-byte global load of row g (and g+8) at
// k-offset t*8 inside a 32-wide k block *is* its A fragment for two consecutive instructions, because the k order
// inside a block may be permuted freely as long as the B fragment uses the same permutation — and the matching B
// fragment is the 16 bytes of activation row (n0+g) at the same k-offset, read from a shared-memory tile.
// CTA = 8 warps = (8/KS) tiles of 16 weight rows x KS interleaved slices of every k tile; the K-slices meet in shared
// memory at the end.  Activation k tiles stream through a double-buffered, bank-conflict-free shared-memory ring with
// cp.async.  Products are exact; the tensor-core accumulation order differs from the reference's sequential fp32
// sum (jsgrad/tensor.ts:2593-2605), like every other reduction on this device.
//
// int8 weights (Int8Linear, jsgrad/models/llama3.ts:35): a lane's 16-byte load holds 16 weights, which it turns into
// fp16 as half(q) * scale[row] (one rounding, as the reference's dequantised matrix) for four instructions; the k block
// is then 64 wide and the matching activation chunk 32 bytes.
//
// Epilogues: STORE, RESIDUAL (fp16 add), SWIGLU (two matrices, silu(gate)*up, jsgrad/models/llama.ts:108-110),
// LOGITS (store + per-row (value, lowest index) key, jsgrad/tensor.ts:2314-2320).
#include <stdlib.h>

#include "common.cuh"
#include "transcendental.cuh"

enum { GS_STORE = 0, GS_RESIDUAL = 1, GS_SWIGLU = 2, GS_LOGITS = 3, GS_PARTIAL = 4 };

struct GemmSmallArgs {
  const __half* x;   // [M][K]
  const void* w0;    // [N][K] fp16, or int8 with per-row scales s0
  const void* w1;    // SWIGLU: up projection
  const __half* s0;  // [N] (int8 weights)
  const __half* s1;
  __half* y;         // [M][N]
  const __half* residual;
  unsigned long long* key;  // [M] (LOGITS)
  float* y32;               // [M][N] unrounded sums (PARTIAL)
  int M, N, K, row_offset;
  int w_late;  // the weights were written by the preceding kernel: no load before the dependency wait
};

constexpr int GS_THREADS = 256;
constexpr int GS_WARPS = 8;
constexpr int GS_KT = 512;                 // activation k tile (halves)
constexpr int GS_ROW_BYTES = GS_KT * 2 + 64;  // padded row: rows g and g+1 land 4 x 16 B apart modulo 128 B
constexpr int GS_ROW_BYTES_W8 = GS_KT * 2 + 16;  // int8 weights read 32 B per lane: rows g and g+1 land 16 B apart

// int8 x16 (one uint4) -> eight half2 words of half(q) * s in k order, each product rounded once.  Bytes become halves
// exactly through the 0x6400 (1024.0) exponent trick.
__device__ __forceinline__ void dequant16_h2(const uint4& raw, __half2 s2, uint32_t (&out)[8]) {
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);  // 1024 + 128
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t v = words[i] ^ 0x80808080u;                  // signed -> offset-binary
    uint32_t lo = __byte_perm(v, 0x64646464u, 0x4140);          // bytes 0,1 -> halves 0x64b0, 0x64b1
    uint32_t hi = __byte_perm(v, 0x64646464u, 0x4342);          // bytes 2,3
    const __half2 a = __hmul2_rn(__hsub2(*reinterpret_cast<__half2*>(&lo), bias), s2);
    const __half2 b = __hmul2_rn(__hsub2(*reinterpret_cast<__half2*>(&hi), bias), s2);
    out[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
    out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
  }
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// D (16x8, fp32) += A (16x16, fp16, row) * B (16x8, fp16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, int KS, int EPI, bool W8>
__global__ void __launch_bounds__(GS_THREADS, (MT <= 32 ? 2 : 1)) gemm_small_kernel(const GemmSmallArgs a) {
  constexpr int KBLK = W8 ? 64 : 32;         // k block: 4 lanes x one 16-byte weight load each
  constexpr int CH = KBLK / 4;               // weights per lane and block
  constexpr int ROWB = W8 ? GS_ROW_BYTES_W8 : GS_ROW_BYTES;
  constexpr int WB = W8 ? 1 : 2;             // bytes per weight
  constexpr int NT = MT / 8;                 // 8-row activation tiles
  constexpr int NW = (EPI == GS_SWIGLU) ? 2 : 1;
  constexpr int TILES = GS_WARPS / KS;       // 16-row weight tiles per CTA
  constexpr int KW = GS_KT / KS;             // k elements of a tile handled by one warp
  constexpr int NBMAX = (NW == 2) ? 4 : 8;   // k blocks whose weight fragments a lane holds at once
  constexpr int NB = (KW / KBLK) < NBMAX ? (KW / KBLK) : NBMAX;
  constexpr int SPT = (KW / KBLK) / NB;      // steps per k tile
  static_assert(NB >= 1 && SPT >= 1 && SPT * NB * KBLK == KW, "k tiling");
  extern __shared__ __align__(16) unsigned char smem[];  // 2 x [MT][GS_ROW_BYTES] activation tiles, then K-slice partials
  __shared__ unsigned long long s_best[GS_WARPS][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile = warp / KS, ks = warp % KS;
  const int K = a.K, N = a.N, M = a.M;
  const int n_kt = (K + GS_KT - 1) / GS_KT;
  pdl_launch();

  const int row0 = (blockIdx.x * TILES + tile) * 16;  // first weight row of this warp's tile
  const bool tile_ok = row0 < N;
  const int ra = min(row0 + g, N - 1), rb = min(row0 + g + 8, N - 1);  // clamp: duplicates are never stored
  const unsigned char* wa[NW];
  const unsigned char* wb[NW];
  wa[0] = (const unsigned char*)a.w0 + (size_t)ra * K * WB; wb[0] = (const unsigned char*)a.w0 + (size_t)rb * K * WB;
  if (NW == 2) { wa[NW - 1] = (const unsigned char*)a.w1 + (size_t)ra * K * WB; wb[NW - 1] = (const unsigned char*)a.w1 + (size_t)rb * K * WB; }
  __half2 sa[NW], sb[NW];  // per-row scales of int8 weights
  if (W8) {
    sa[0] = __half2half2(a.s0[ra]); sb[0] = __half2half2(a.s0[rb]);
    if (NW == 2) { sa[NW - 1] = __half2half2(a.s1[ra]); sb[NW - 1] = __half2half2(a.s1[rb]); }
  }

  float acc[NW][NT][4];
#pragma unroll
  for (int w = 0; w < NW; w++)
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) acc[w][j][i] = 0.f;

  // weights of k tile 0 are requested before the dependency wait: they do not depend on the previous kernel
  uint4 fa[NW][NB], fb[NW][NB];
  auto load_w = [&](int kt, int sp) {
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const int k = kt * GS_KT + ks * KW + (sp * NB + b) * KBLK + t * CH;
      const bool ok = tile_ok && (k + CH <= K);
#pragma unroll
      for (int w = 0; w < NW; w++) {
        fa[w][b] = ok ? ld_stream_128(wa[w] + (size_t)k * WB) : make_uint4(0, 0, 0, 0);
        fb[w][b] = ok ? ld_stream_128(wb[w] + (size_t)k * WB) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  if (!a.w_late) load_w(0, 0);
  pdl_wait();
  if (a.w_late) load_w(0, 0);

  // activation tile loader: MT rows x GS_KT halves, 16 bytes per cp.async, zero fill past M or K
  auto load_x = [&](int kt, int bufi) {
    unsigned char* dst = smem + (size_t)bufi * MT * ROWB;
    for (int c = tid; c < MT * (GS_KT / 8); c += GS_THREADS) {
      const int m = c / (GS_KT / 8), kc = c % (GS_KT / 8);
      const int k = kt * GS_KT + kc * 8;
      unsigned char* d = dst + (size_t)m * ROWB + (size_t)kc * 16;
      if (m < M && k + 8 <= K) cp_async_16(d, a.x + (size_t)m * K + k);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };
  load_x(0, 0);

  for (int kt = 0; kt < n_kt; kt++) {
    const int cur = kt & 1;
    if (kt + 1 < n_kt) {
      load_x(kt + 1, cur ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const unsigned char* xs = smem + (size_t)cur * MT * ROWB;
    for (int sp = 0; sp < SPT; sp++) {
#pragma unroll
      for (int b = 0; b < NB; b++) {
        // byte offset of this lane's 16 bytes inside an activation row
        const int koff = (ks * KW + (sp * NB + b) * KBLK + t * CH) * 2;
        if (!W8) {
#pragma unroll
          for (int j = 0; j < NT; j++) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)(j * 8 + g) * ROWB + koff);
#pragma unroll
            for (int w = 0; w < NW; w++) {
              // first instruction: halves 0-3 of the chunk (k 2t,2t+1 | 2t+8,2t+9 of the permuted block), second: 4-7
              mma_16816(acc[w][j], fa[w][b].x, fb[w][b].x, fa[w][b].y, fb[w][b].y, xv.x, xv.y);
              mma_16816(acc[w][j], fa[w][b].z, fb[w][b].z, fa[w][b].w, fb[w][b].w, xv.z, xv.w);
            }
          }
        } else {
          uint32_t da[NW][8], db[NW][8];  // the lane's 16 weights of rows g and g+8 as fp16 pairs
#pragma unroll
          for (int w = 0; w < NW; w++) { dequant16_h2(fa[w][b], sa[w], da[w]); dequant16_h2(fb[w][b], sb[w], db[w]); }
#pragma unroll
          for (int j = 0; j < NT; j++) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)(j * 8 + g) * ROWB + koff);
            const uint4 x0 = xp[0], x1 = xp[1];
            const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
              for (int i = 0; i < 4; i++)  // instruction i: halves 4i .. 4i+3 of the chunk
                mma_16816(acc[w][j], da[w][2 * i], db[w][2 * i], da[w][2 * i + 1], db[w][2 * i + 1], xw[2 * i], xw[2 * i + 1]);
          }
        }
      }
      if (sp + 1 < SPT) load_w(kt, sp + 1);
      else if (kt + 1 < n_kt) load_w(kt + 1, 0);
    }
    __syncthreads();  // the buffer read above is refilled by the next iteration's cp.async
  }

  // ---- fold the K slices (fixed order) through shared memory; slice 0 of every tile keeps the result
  if (KS > 1) {
    float* part = reinterpret_cast<float*>(smem);  // [TILES][KS][NW*NT*4][32]; the activation tiles are dead now
    constexpr int PER = NW * NT * 4;
    float* mine = part + ((size_t)(tile * KS + ks) * PER) * 32;
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) mine[(size_t)((w * NT + j) * 4 + i) * 32 + lane] = acc[w][j][i];
    __syncthreads();
    if (ks == 0) {
#pragma unroll
      for (int w = 0; w < NW; w++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int i = 0; i < 4; i++) {
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < KS; q++) s += part[((size_t)(tile * KS + q) * PER + (size_t)((w * NT + j) * 4 + i)) * 32 + lane];
            acc[w][j][i] = s;
          }
    }
  }

  // ---- epilogue: accumulator i of tile j is (weight row g + 8*(i/2), activation row 8j + 2t + (i%2))
  unsigned long long best[NT][2];
#pragma unroll
  for (int j = 0; j < NT; j++) { best[j][0] = 0ull; best[j][1] = 0ull; }
  if (ks == 0 && tile_ok) {
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int row = row0 + g + 8 * (i >> 1), m = j * 8 + 2 * t + (i & 1);
        if (row < N && m < M) {
          const size_t o = (size_t)m * N + row;
          if (EPI == GS_PARTIAL) { a.y32[o] = acc[0][j][i]; continue; }
          __half v = __float2half_rn(acc[0][j][i]);
          if (EPI == GS_RESIDUAL) v = hadd1(a.residual[o], v);
          if (EPI == GS_SWIGLU) v = jg_silu_mul(v, __float2half_rn(acc[NW - 1][j][i]));
          a.y[o] = v;
          if (EPI == GS_LOGITS) {
            const unsigned long long k = argmax_key(v, (uint32_t)(row + a.row_offset));
            best[j][i & 1] = k > best[j][i & 1] ? k : best[j][i & 1];
          }
        }
      }
  }
  if (EPI == GS_LOGITS) {
    // lanes with the same t hold the same activation rows: fold over g, then one atomic per row and warp
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        unsigned long long b = best[j][e];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
          b = other > b ? other : b;
        }
        const int m = j * 8 + 2 * t + e;
        if (g == 0 && m < M && b != 0ull) atomicMax(a.key + m, b);
      }
    (void)s_best;
  }
}

// ------------------------------------------------------------------------------------------------ host side
template <int MT, int KS, int EPI, bool W8>
static int launch_gs(jg_dev* dev, const GemmSmallArgs& a, const char* name) {
  auto kern = gemm_small_kernel<MT, KS, EPI, W8>;
  constexpr int NW = (EPI == GS_SWIGLU) ? 2 : 1;
  const size_t x_bytes = (size_t)2 * MT * (W8 ? GS_ROW_BYTES_W8 : GS_ROW_BYTES);
  const size_t p_bytes = KS > 1 ? (size_t)GS_WARPS * NW * (MT / 8) * 4 * 32 * sizeof(float) : 0;
  const size_t smem = x_bytes > p_bytes ? x_bytes : p_bytes;
  static bool attr_set[8] = {false, false, false, false, false, false, false, false};
  const int slot = dev->ordinal & 7;
  if (!attr_set[slot] && smem > 48 * 1024) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[slot] = true;
  }
  const int rows_per_cta = (GS_WARPS / KS) * 16;
  const unsigned blocks = (unsigned)((a.N + rows_per_cta - 1) / rows_per_cta);
  return jg_launch(dev, name, kern, dim3(blocks), dim3(GS_THREADS), smem, a);
}

template <int MT, int EPI, bool W8>
static int dispatch_ks(jg_dev* dev, const GemmSmallArgs& a, const char* name) {
  // enough CTAs to fill the machine twice over: 16-row tiles x K slices >= 2 x 8 warps x SMs
  const long long tiles = (a.N + 15) / 16;
  const long long want = 2LL * GS_WARPS * dev->sm_count;
  if (tiles >= want || a.K < 8 * 256) return launch_gs<MT, 1, EPI, W8>(dev, a, name);
  if (tiles * 2 >= want) return launch_gs<MT, 2, EPI, W8>(dev, a, name);
  if (tiles * 4 >= want) return launch_gs<MT, 4, EPI, W8>(dev, a, name);
  return launch_gs<MT, 8, EPI, W8>(dev, a, name);
}

template <int EPI, bool W8>
static int dispatch_mt(jg_dev* dev, const GemmSmallArgs& a, const char* name) {
  if (a.M <= 8) return dispatch_ks<8, EPI, W8>(dev, a, name);
  if (a.M <= 16) return dispatch_ks<16, EPI, W8>(dev, a, name);
  if (a.M <= 32) return dispatch_ks<32, EPI, W8>(dev, a, name);
  if (a.M <= 64) return dispatch_ks<64, EPI, W8>(dev, a, name);
  jg_set_error("%s: M=%d rows is beyond the small-batch projection kernels (max 64 per call)", name, a.M);
  return JG_ENOTSUP;
}

template <bool W8>
static int dispatch_epi(jg_dev* dev, int epi, const GemmSmallArgs& a) {
  switch (epi) {
    case GS_STORE: return dispatch_mt<GS_STORE, W8>(dev, a, "linear");
    case GS_RESIDUAL: return dispatch_mt<GS_RESIDUAL, W8>(dev, a, "linear");
    case GS_SWIGLU: return dispatch_mt<GS_SWIGLU, W8>(dev, a, "norm_swiglu");
    case GS_LOGITS: return dispatch_mt<GS_LOGITS, W8>(dev, a, "norm_logits_argmax");
    case GS_PARTIAL: return dispatch_mt<GS_PARTIAL, W8>(dev, a, "linear_partial");
  }
  jg_set_error("projection: unknown epilogue %d", epi);
  return JG_EINVAL;
}

// Entry used by gemv.cu's public functions for up to 64 rows; s0 / s1 non-null = int8 weights with per-row scales.
int jg_gemm_small(jg_dev* dev, int epi, const void* x, const void* w0, const void* w1, const void* s0, const void* s1,
                  void* y, const void* residual, void* key, int M, int N, int K, int row_offset) {
  JG_REQUIRE(K % (s0 ? 16 : 8) == 0, "projection: K=%d must be a multiple of %d", K, s0 ? 16 : 8);
  GemmSmallArgs a = {};
  a.x = (const __half*)x; a.w0 = w0; a.w1 = w1; a.s0 = (const __half*)s0; a.s1 = (const __half*)s1; a.y = (__half*)y;
  a.residual = (const __half*)residual; a.key = (unsigned long long*)key; a.M = M; a.N = N; a.K = K;
  a.row_offset = row_offset;
  a.w_late = jg_is_fresh(dev, w0) || jg_is_fresh(dev, w1);
  if (epi == GS_PARTIAL) { a.y = nullptr; a.y32 = (float*)y; }
  return s0 ? dispatch_epi<true>(dev, epi, a) : dispatch_epi<false>(dev, epi, a);
}
