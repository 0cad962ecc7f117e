// Weight-streaming matrix-vector kernels for decode (M = batch rows <= 8): y[m][n] = sum_k x[m][k] * W[n][k].
//
// The weight matrix is read exactly once per launch with 128-bit streaming loads; the activation rows live in
// shared memory.  A warp owns RW consecutive output rows at a time and walks K with U independent 16-byte loads
// per lane and row in flight, so that one SM keeps tens of KB outstanding towards HBM.  Products of fp16 operands
// are exact in fp32 and are accumulated in fp32 (Tensor.dot with sum_acc_dtype: jsgrad/tensor.ts:2593-2605,
// jsgrad/dtype.ts:243-248); only the summation order differs from a sequential loop.
//
// Fused around the reduction, all from the Llama block (jsgrad/models/llama.ts:108-127,210):
//   prologue  NORM      x <- RMSNorm(x) * g            (jsgrad/nn/index.ts:586-588)
//   epilogue  RESIDUAL  y <- residual + half(acc)       (x.add(...), fp16 add)
//             SWIGLU    y <- silu(half(acc_gate)) * half(acc_up)
//             LOGITS    y <- half(acc) and (value, lowest index) folded into a 64-bit max key per row
#include "common.cuh"
#include "transcendental.cuh"

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_LOGITS = 3 };

struct GemvArgs {
  const __half* x;       // [M][K]
  const __half* norm_w;  // [K] (NORM only)
  const void* w0;        // [N][K] fp16 or int8
  const void* w1;        // second matrix (SWIGLU: up projection)
  const __half* s0;      // [N] int8 scales
  const __half* s1;
  __half* y;             // [M][N]
  const __half* residual;
  unsigned long long* key;  // [M] (LOGITS)
  float eps, recip_k;
  int M, N, K;
};

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

// int8 x16 (one uint4) -> sixteen fp32 values of half(q) * s, the fp16 product rounded once (Int8Linear:
// jsgrad/models/llama3.ts:35).  Bytes are turned into halves exactly through the 0x6400 (1024.0) exponent trick.
__device__ __forceinline__ void dequant16(const uint4& raw, __half2 s2, float (&w)[16]) {
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);  // 1024 + 128
#pragma unroll
  for (int i = 0; i < 4; i++) {
    uint32_t v = words[i] ^ 0x80808080u;                  // signed -> offset-binary
    uint32_t lo = __byte_perm(v, 0x64646464u, 0x4140);    // bytes 0,1 -> halves 0x64b0, 0x64b1
    uint32_t hi = __byte_perm(v, 0x64646464u, 0x4342);    // bytes 2,3
    __half2 a = __hsub2(*reinterpret_cast<__half2*>(&lo), bias);  // exact: integers below 2048
    __half2 b = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
    float2 fa = __half22float2(__hmul2_rn(a, s2));
    float2 fb = __half22float2(__hmul2_rn(b, s2));
    w[i * 4 + 0] = fa.x; w[i * 4 + 1] = fa.y; w[i * 4 + 2] = fb.x; w[i * 4 + 3] = fb.y;
  }
}

template <int MT, bool W8, int EPI, bool NORM, int RW, int U>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);  // [MT][K]
  __shared__ float red[GEMV_WARPS];
  __shared__ float s_rs;
  constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
  constexpr int CH = W8 ? 16 : 8;  // weights per 16-byte load
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.K, N = a.N;

  // ---- prologue: activation rows -> shared memory (normalised when NORM); rows beyond M are zero
  for (int m = 0; m < MT; m++) {
    __half* xm = xs + (size_t)m * K;
    if (m >= a.M) {
      for (int c = tid; c < K / 8; c += GEMV_THREADS) reinterpret_cast<uint4*>(xm)[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const __half* xg = a.x + (size_t)m * K;
    if (NORM) {
      float ss = 0.f;
      for (int c = tid; c < K / 8; c += GEMV_THREADS) {
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
        float t = 0.f;
        for (int i = 0; i < GEMV_WARPS; i++) t += red[i];
        s_rs = sqrtf(__fdiv_rn(1.0f, __fadd_rn(__fmul_rn(t, a.recip_k), a.eps)));
      }
      __syncthreads();
      const float rs = s_rs;
      for (int c = tid; c < K / 8; c += GEMV_THREADS) {
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
      for (int c = tid; c < K / 8; c += GEMV_THREADS) reinterpret_cast<uint4*>(xm)[c] = ld_128(xg + (size_t)c * 8);
    }
  }
  __syncthreads();

  // ---- main loop: contiguous, balanced slice of row groups per warp
  const long long gw = (long long)blockIdx.x * GEMV_WARPS + warp, GW = (long long)gridDim.x * GEMV_WARPS;
  const int n_units = (N + RW - 1) / RW;
  const int u_begin = (int)(gw * n_units / GW), u_end = (int)((gw + 1) * n_units / GW);
  const int KC = K / CH;  // 16-byte chunks per weight row
  const size_t row_bytes = W8 ? (size_t)K : (size_t)K * 2;
  unsigned long long best[MT];
  if (EPI == EPI_LOGITS) {
#pragma unroll
    for (int m = 0; m < MT; m++) best[m] = 0ull;
  }

  for (int unit = u_begin; unit < u_end; unit++) {
    const int r0 = unit * RW;
    float acc[NW][RW][MT];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
      for (int r = 0; r < RW; r++)
#pragma unroll
        for (int m = 0; m < MT; m++) acc[w][r][m] = 0.f;

    const unsigned char* wrow[NW][RW];
    __half2 sc[NW][RW];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
      for (int r = 0; r < RW; r++) {
        const int row = (r0 + r < N) ? (r0 + r) : (N - 1);  // clamp: duplicates are never stored
        wrow[w][r] = reinterpret_cast<const unsigned char*>(w == 0 ? a.w0 : a.w1) + (size_t)row * row_bytes;
        if (W8) sc[w][r] = __half2half2((w == 0 ? a.s0 : a.s1)[row]);
      }

    for (int c0 = lane; c0 < KC; c0 += 32 * U) {
      uint4 wv[NW][RW][U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int c = c0 + 32 * u;
        const bool ok = c < KC;
#pragma unroll
        for (int w = 0; w < NW; w++)
#pragma unroll
          for (int r = 0; r < RW; r++)
            wv[w][r][u] = ok ? ld_stream_128(wrow[w][r] + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int c = c0 + 32 * u;
        if (c >= KC) break;
        if (!W8) {
#pragma unroll
          for (int m = 0; m < MT; m++) {
            float xf[8];
            unpack8(*reinterpret_cast<const uint4*>(xs + (size_t)m * K + (size_t)c * 8), xf);
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
              for (int r = 0; r < RW; r++) acc[w][r][m] = dot8_acc(acc[w][r][m], wv[w][r][u], xf);
          }
        } else {
          float wf[NW][RW][16];
#pragma unroll
          for (int w = 0; w < NW; w++)
#pragma unroll
            for (int r = 0; r < RW; r++) dequant16(wv[w][r][u], sc[w][r], wf[w][r]);
#pragma unroll
          for (int m = 0; m < MT; m++) {
            float xf[16];
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * K + (size_t)c * 16);
            {
              float lo[8], hi[8];
              unpack8(xp[0], lo);
              unpack8(xp[1], hi);
#pragma unroll
              for (int k = 0; k < 8; k++) { xf[k] = lo[k]; xf[8 + k] = hi[k]; }
            }
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
              for (int r = 0; r < RW; r++)
#pragma unroll
                for (int k = 0; k < 16; k++) acc[w][r][m] = fmaf(wf[w][r][k], xf[k], acc[w][r][m]);
          }
        }
      }
    }

    // ---- reduce across the warp and apply the epilogue; lane (r*MT + m) stores output (row r0+r, m)
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
      for (int r = 0; r < RW; r++)
#pragma unroll
        for (int m = 0; m < MT; m++) acc[w][r][m] = warp_sum(acc[w][r][m]);

#pragma unroll
    for (int r = 0; r < RW; r++)
#pragma unroll
      for (int m = 0; m < MT; m++) {
        if (lane == ((r * MT + m) & 31) && r0 + r < N && m < a.M) {
          const size_t o = (size_t)m * N + (size_t)(r0 + r);
          __half v = __float2half_rn(acc[0][r][m]);
          if (EPI == EPI_RESIDUAL) v = hadd1(a.residual[o], v);
          if (EPI == EPI_SWIGLU) v = jg_silu_mul(v, __float2half_rn(acc[NW - 1][r][m]));
          a.y[o] = v;
          if (EPI == EPI_LOGITS) {
            unsigned long long k = argmax_key(v, (uint32_t)(r0 + r));
            best[m] = k > best[m] ? k : best[m];
          }
        }
      }
  }

  if (EPI == EPI_LOGITS) {
#pragma unroll
    for (int m = 0; m < MT; m++) {
      unsigned long long b = best[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
        b = other > b ? other : b;
      }
      if (lane == 0 && m < a.M && b != 0ull) atomicMax(a.key + m, b);
    }
  }
}

// ------------------------------------------------------------------------------------------------ host side
template <int MT, bool W8, int EPI, bool NORM>
static int launch_gemv(jg_dev* dev, const GemvArgs& a, const char* name) {
  // RW x U 16-byte loads per lane in flight; SWIGLU streams two matrices, so it takes half the rows per pass.
  constexpr int RW = (EPI == EPI_SWIGLU) ? 1 : 2;
  constexpr int U = (MT >= 4 || W8) ? 2 : 4;
  auto kern = gemv_kernel<MT, W8, EPI, NORM, RW, U>;
  const size_t smem = (size_t)MT * a.K * sizeof(__half);
  if (smem + 1024 > (size_t)dev->prop.sharedMemPerBlockOptin) {
    jg_set_error("%s: %d activation rows of K=%d need %zu B of shared memory (limit %zu)", name, MT, a.K, smem,
                 (size_t)dev->prop.sharedMemPerBlockOptin);
    return JG_ENOTSUP;
  }
  static size_t smem_set[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int slot = dev->ordinal & 7;
  if (smem > 48 * 1024 && smem > smem_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev->prop.sharedMemPerBlockOptin - 1024));
    smem_set[slot] = dev->prop.sharedMemPerBlockOptin;
  }
  int occ = 0;
  JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, GEMV_THREADS, smem));
  if (occ < 1) occ = 1;
  if (occ > 4) occ = 4;
  const int n_units = (a.N + RW - 1) / RW;
  long long blocks = (long long)dev->sm_count * occ;
  const long long max_useful = (n_units + GEMV_WARPS - 1) / GEMV_WARPS;
  if (blocks > max_useful) blocks = max_useful;
  if (blocks < 1) blocks = 1;
  kern<<<(unsigned)blocks, GEMV_THREADS, smem, dev->stream>>>(a);
  return jg_after_launch(dev, name);
}

template <bool W8, int EPI, bool NORM>
static int dispatch_m(jg_dev* dev, const GemvArgs& a, const char* name) {
  if (a.M == 1) return launch_gemv<1, W8, EPI, NORM>(dev, a, name);
  if (a.M == 2) return launch_gemv<2, W8, EPI, NORM>(dev, a, name);
  if (a.M <= 4) return launch_gemv<4, W8, EPI, NORM>(dev, a, name);
  if (a.M <= 8) return launch_gemv<8, W8, EPI, NORM>(dev, a, name);
  jg_set_error("%s: M=%d rows is beyond the matrix-vector kernels (max 8)", name, a.M);
  return JG_ENOTSUP;
}

static int check_common(const char* name, uint64_t y, uint64_t x, uint64_t w, uint64_t scale, int M, int N, int K) {
  JG_REQUIRE(M > 0 && N > 0 && K > 0, "%s: bad shape M=%d N=%d K=%d", name, M, N, K);
  JG_REQUIRE(K % (scale ? 16 : 8) == 0, "%s: K=%d must be a multiple of %d", name, K, scale ? 16 : 8);
  JG_REQUIRE(jg_aligned(y, 2) && jg_aligned(x, 16) && jg_aligned(w, 16), "%s: null or misaligned pointer", name);
  JG_REQUIRE(scale == 0 || jg_aligned(scale, 2), "%s: misaligned scale pointer", name);
  return JG_OK;
}

JG_API int jg_linear(jg_dev* dev, uint64_t y, uint64_t x, uint64_t w, uint64_t scale, uint64_t residual, int32_t M,
                     int32_t N, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("linear", y, x, w, scale, M, N, K);
  if (rc) return rc;
  GemvArgs a = {};
  a.x = (const __half*)x; a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)y;
  a.residual = (const __half*)residual; a.M = M; a.N = N; a.K = K;
  if (residual) {
    JG_REQUIRE(jg_aligned(residual, 2), "linear: misaligned residual pointer");
    return scale ? dispatch_m<true, EPI_RESIDUAL, false>(dev, a, "linear") : dispatch_m<false, EPI_RESIDUAL, false>(dev, a, "linear");
  }
  return scale ? dispatch_m<true, EPI_STORE, false>(dev, a, "linear") : dispatch_m<false, EPI_STORE, false>(dev, a, "linear");
}

JG_API int jg_norm_linear(jg_dev* dev, uint64_t y, uint64_t x, uint64_t norm_w, float eps, uint64_t w, uint64_t scale,
                          int32_t M, int32_t N, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("norm_linear", y, x, w, scale, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(norm_w, 16), "norm_linear: null or misaligned norm weight");
  GemvArgs a = {};
  a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.eps = eps; a.recip_k = (float)(1.0 / (double)K);
  a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)y; a.M = M; a.N = N; a.K = K;
  return scale ? dispatch_m<true, EPI_STORE, true>(dev, a, "norm_linear") : dispatch_m<false, EPI_STORE, true>(dev, a, "norm_linear");
}

JG_API int jg_norm_swiglu(jg_dev* dev, uint64_t y, uint64_t x, uint64_t norm_w, float eps, uint64_t w_gate,
                          uint64_t s_gate, uint64_t w_up, uint64_t s_up, int32_t M, int32_t N, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("norm_swiglu", y, x, w_gate, s_gate, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(w_up, 16), "norm_swiglu: null or misaligned up-projection weight");
  JG_REQUIRE((s_gate == 0) == (s_up == 0), "norm_swiglu: gate and up projections must share a weight format");
  GemvArgs a = {};
  a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.eps = eps; a.recip_k = (float)(1.0 / (double)K);
  a.w0 = (const void*)w_gate; a.w1 = (const void*)w_up; a.s0 = (const __half*)s_gate; a.s1 = (const __half*)s_up;
  a.y = (__half*)y; a.M = M; a.N = N; a.K = K;
  if (norm_w) {
    JG_REQUIRE(jg_aligned(norm_w, 16), "norm_swiglu: misaligned norm weight");
    return s_gate ? dispatch_m<true, EPI_SWIGLU, true>(dev, a, "norm_swiglu") : dispatch_m<false, EPI_SWIGLU, true>(dev, a, "norm_swiglu");
  }
  return s_gate ? dispatch_m<true, EPI_SWIGLU, false>(dev, a, "norm_swiglu") : dispatch_m<false, EPI_SWIGLU, false>(dev, a, "norm_swiglu");
}

JG_API int jg_norm_logits_argmax(jg_dev* dev, uint64_t logits, uint64_t key, uint64_t x, uint64_t norm_w, float eps,
                                 uint64_t w, uint64_t scale, int32_t M, int32_t V, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("norm_logits_argmax", logits, x, w, scale, M, V, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(norm_w, 16) && jg_aligned(key, 8), "norm_logits_argmax: null or misaligned pointer");
  GemvArgs a = {};
  a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.eps = eps; a.recip_k = (float)(1.0 / (double)K);
  a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)logits; a.key = (unsigned long long*)key;
  a.M = M; a.N = V; a.K = K;
  return scale ? dispatch_m<true, EPI_LOGITS, true>(dev, a, "norm_logits_argmax") : dispatch_m<false, EPI_LOGITS, true>(dev, a, "norm_logits_argmax");
}
