// Small HBM-bound kernels of the Llama forward: embedding gather, RMSNorm, RoPE table, SwiGLU product, argmax,
// and the seeded synthetic-tensor fills.  Each is one pass over its data with 128-bit accesses where the shape
// allows it.
#include <math.h>

#include "common.cuh"
#include "transcendental.cuh"

// ------------------------------------------------------------------------------------------------ embedding
// Embedding.call == row gather (jsgrad/nn/index.ts:607-619): out[i,:] = W[tokens[i],:].
__global__ void embed_f16_kernel(__half* __restrict__ out, const int32_t* __restrict__ tokens,
                                 const __half* __restrict__ w, int n_tok, int dim, int vocab) {
  pdl_launch();
  pdl_wait();
  const int per_row = dim / 8;
  for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < (long long)n_tok * per_row;
       it += (long long)gridDim.x * blockDim.x) {
    int i = (int)(it / per_row), c = (int)(it % per_row);
    const int tok = tokens[i];
    // an index outside the table matches no one-hot row: the reference's sum is zero there
    reinterpret_cast<uint4*>(out + (size_t)i * dim)[c] =
        (tok >= 0 && tok < vocab) ? ld_128(w + (size_t)tok * dim + (size_t)c * 8) : make_uint4(0, 0, 0, 0);
  }
}
// Int8Embedding.call (jsgrad/models/llama3.ts:71-77): out[i,k] = half(Wq[tok,k]) * scale[tok] (fp16 product).
__global__ void embed_w8_kernel(__half* __restrict__ out, const int32_t* __restrict__ tokens,
                                const int8_t* __restrict__ wq, const __half* __restrict__ scale, int n_tok, int dim,
                                int vocab) {
  pdl_launch();
  pdl_wait();
  const int per_row = dim / 8;
  for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < (long long)n_tok * per_row;
       it += (long long)gridDim.x * blockDim.x) {
    int i = (int)(it / per_row), c = (int)(it % per_row);
    const int tok = tokens[i];
    if (tok < 0 || tok >= vocab) {
      reinterpret_cast<uint4*>(out + (size_t)i * dim)[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const __half s = scale[tok];
    uint2 raw = *reinterpret_cast<const uint2*>(wq + (size_t)tok * dim + (size_t)c * 8);
    const int8_t* q = reinterpret_cast<const int8_t*>(&raw);
    __align__(16) __half o[8];
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = hmul1(__int2half_rn((int)q[k]), s);
    reinterpret_cast<uint4*>(out + (size_t)i * dim)[c] = *reinterpret_cast<uint4*>(o);
  }
}

JG_API int jg_embed(jg_dev* dev, uint64_t out, uint64_t tokens, uint64_t w, uint64_t scale, int32_t n_tok, int32_t dim,
                    int32_t vocab) {
  JG_ENTER(dev);
  JG_REQUIRE(n_tok > 0 && dim > 0 && vocab > 0 && dim % 8 == 0, "embed: bad shape n_tok=%d dim=%d vocab=%d", n_tok, dim, vocab);
  JG_REQUIRE(jg_aligned(out, 16) && jg_aligned(w, 16) && jg_aligned(tokens, 4), "embed: null or misaligned pointer");
  long long items = (long long)n_tok * (dim / 8);
  int blocks = (int)((items + 255) / 256);
  if (blocks > dev->sm_count * 8) blocks = dev->sm_count * 8;
  if (scale == 0)
    return jg_launch(dev, "embed", embed_f16_kernel, dim3(blocks), dim3(256), 0, (__half*)out, (const int32_t*)tokens,
                     (const __half*)w, n_tok, dim, vocab);
  return jg_launch(dev, "embed", embed_w8_kernel, dim3(blocks), dim3(256), 0, (__half*)out, (const int32_t*)tokens,
                   (const int8_t*)w, (const __half*)scale, n_tok, dim, vocab);
}

// ------------------------------------------------------------------------------------------------ RMSNorm
// RMSNorm.call (jsgrad/nn/index.ts:586-588): y = half(float(x) * sqrt(1/(mean(x^2)+eps))) * w, one CTA per row.
__global__ void __launch_bounds__(256) rmsnorm_kernel(__half* __restrict__ y, const __half* __restrict__ x,
                                                      const __half* __restrict__ w, int dim, float eps, float recip_d) {
  __shared__ float red[8];
  __shared__ float s_rs;
  const int row = blockIdx.x;
  const __half* xr = x + (size_t)row * dim;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dim / 8; c += 256) {
    float v[8];
    unpack8(ld_128(xr + (size_t)c * 8), v);
#pragma unroll
    for (int k = 0; k < 8; k++) ss = fmaf(v[k], v[k], ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; i++) t += red[i];
    s_rs = sqrtf(__fdiv_rn(1.0f, __fadd_rn(__fmul_rn(t, recip_d), eps)));
  }
  __syncthreads();
  const float rs = s_rs;
  for (int c = threadIdx.x; c < dim / 8; c += 256) {
    float v[8];
    unpack8(ld_128(xr + (size_t)c * 8), v);
    uint4 wv = ld_128(w + (size_t)c * 8);
    const __half* wh = reinterpret_cast<const __half*>(&wv);
    __align__(16) __half o[8];
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = hmul1(__float2half_rn(__fmul_rn(v[k], rs)), wh[k]);
    reinterpret_cast<uint4*>(y + (size_t)row * dim)[c] = *reinterpret_cast<uint4*>(o);
  }
}

JG_API int jg_rmsnorm(jg_dev* dev, uint64_t y, uint64_t x, uint64_t w, int32_t rows, int32_t dim, float eps) {
  JG_ENTER(dev);
  JG_REQUIRE(rows > 0 && dim > 0 && dim % 8 == 0, "rmsnorm: bad shape rows=%d dim=%d", rows, dim);
  JG_REQUIRE(jg_aligned(y, 16) && jg_aligned(x, 16) && jg_aligned(w, 16), "rmsnorm: null or misaligned pointer");
  rmsnorm_kernel<<<rows, 256, 0, dev->stream>>>((__half*)y, (const __half*)x, (const __half*)w, dim, eps,
                                                (float)(1.0 / (double)dim));
  return jg_after_launch(dev, "rmsnorm");
}

// ------------------------------------------------------------------------------------------------ SwiGLU product
__global__ void swiglu_kernel(__half* __restrict__ y, const __half* __restrict__ g, const __half* __restrict__ u, long long n8) {
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < n8; c += (long long)gridDim.x * blockDim.x) {
    uint4 gv = ld_128(g + c * 8), uv = ld_128(u + c * 8);
    const __half* gh = reinterpret_cast<const __half*>(&gv);
    const __half* uh = reinterpret_cast<const __half*>(&uv);
    __align__(16) __half o[8];
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = jg_silu_mul(gh[k], uh[k]);
    reinterpret_cast<uint4*>(y)[c] = *reinterpret_cast<uint4*>(o);
  }
}

JG_API int jg_swiglu(jg_dev* dev, uint64_t y, uint64_t g, uint64_t u, int64_t n) {
  JG_ENTER(dev);
  JG_REQUIRE(n > 0 && n % 8 == 0, "swiglu: element count %lld must be a positive multiple of 8", (long long)n);
  JG_REQUIRE(jg_aligned(y, 16) && jg_aligned(g, 16) && jg_aligned(u, 16), "swiglu: null or misaligned pointer");
  long long n8 = n / 8;
  int blocks = (int)((n8 + 255) / 256);
  if (blocks > dev->sm_count * 8) blocks = dev->sm_count * 8;
  swiglu_kernel<<<blocks, 256, 0, dev->stream>>>((__half*)y, (const __half*)g, (const __half*)u, n8);
  return jg_after_launch(dev, "swiglu");
}

// ------------------------------------------------------------------------------------------------ RoPE table
// precompute_freqs_cis (jsgrad/models/llama.ts:10-14) + the fp16 cast at :205.
// freq_i = 1 / exp2( float(2i) * c ), c = fp32( fp32(1/hd) * ln(theta) * (1/ln 2) ) (constant multiplies fold,
// jsgrad/ops.ts:1363); angle = float(t) * freq_i; cos(x) = sin(pi/2 - x) (jsgrad/tensor.ts:2964-2966).
__global__ void freqs_cis_kernel(__half* __restrict__ table, int half_dim, int end, float c) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)end * half_dim) return;
  int t = (int)(idx / half_dim), i = (int)(idx % half_dim);
  float freq = __fdiv_rn(1.0f, jg_xexp2_f32(__fmul_rn((float)(2 * i), c)));
  float ang = __fmul_rn((float)t, freq);
  float co = jg_xsin_f32(__fsub_rn(1.5707963267948966f, ang));
  float si = jg_xsin_f32(ang);
  table[idx * 2 + 0] = __float2half_rn(co);
  table[idx * 2 + 1] = __float2half_rn(si);
}

JG_API int jg_freqs_cis(jg_dev* dev, uint64_t table, int32_t head_dim, int32_t end, double theta) {
  JG_ENTER(dev);
  JG_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && end > 0 && theta > 0, "freqs_cis: bad arguments");
  JG_REQUIRE(jg_aligned(table, 16), "freqs_cis: null or misaligned pointer");
  float recip_dim = (float)(1.0 / (double)head_dim);
  float c = (float)((double)recip_dim * log(theta) * (1.0 / log(2.0)));
  long long n = (long long)end * (head_dim / 2);
  freqs_cis_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>((__half*)table, head_dim / 2, end, c);
  return jg_after_launch(dev, "freqs_cis");
}

// ------------------------------------------------------------------------------------------------ argmax
// Tensor.argmax (jsgrad/tensor.ts:2314-2320): index of the maximum, lowest index among equals. One CTA per row.
__global__ void __launch_bounds__(256) argmax_kernel(int32_t* __restrict__ out, const __half* __restrict__ x, int n) {
  __shared__ unsigned long long red[8];
  const __half* xr = x + (size_t)blockIdx.x * n;
  unsigned long long best = 0ull;
  for (int i = threadIdx.x; i < n; i += 256) {
    unsigned long long k = argmax_key(xr[i], (uint32_t)i);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; i++) best = red[i] > best ? red[i] : best;
    out[blockIdx.x] = (int32_t)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
  }
}

JG_API int jg_argmax(jg_dev* dev, uint64_t out_idx, uint64_t x, int32_t rows, int32_t n) {
  JG_ENTER(dev);
  JG_REQUIRE(rows > 0 && n > 0, "argmax: bad shape rows=%d n=%d", rows, n);
  JG_REQUIRE(jg_aligned(out_idx, 4) && jg_aligned(x, 2), "argmax: null or misaligned pointer");
  argmax_kernel<<<rows, 256, 0, dev->stream>>>((int32_t*)out_idx, (const __half*)x, n);
  return jg_after_launch(dev, "argmax");
}

__global__ void argmax_finalize_kernel(int32_t* __restrict__ tokens, unsigned long long* __restrict__ key, int M) {
  pdl_launch();
  pdl_wait();
  int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m < M) {
    unsigned long long k = key[m];
    tokens[m] = (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
    key[m] = 0ull;
  }
}

JG_API int jg_argmax_finalize(jg_dev* dev, uint64_t tokens_out, uint64_t key, int32_t M) {
  JG_ENTER(dev);
  JG_REQUIRE(M > 0, "argmax_finalize: bad row count %d", M);
  JG_REQUIRE(jg_aligned(tokens_out, 4) && jg_aligned(key, 8), "argmax_finalize: null or misaligned pointer");
  return jg_launch(dev, "argmax_finalize", argmax_finalize_kernel, dim3((M + 63) / 64), dim3(64), 0, (int32_t*)tokens_out,
                   (unsigned long long*)key, M);
}

__global__ void pos_advance_kernel(int32_t* pos, int B) {
  pdl_launch();
  pdl_wait();
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) pos[b] += 1;
}

JG_API int jg_pos_advance(jg_dev* dev, uint64_t pos, int32_t B) {
  JG_ENTER(dev);
  JG_REQUIRE(B > 0 && jg_aligned(pos, 4), "pos_advance: bad arguments");
  return jg_launch(dev, "pos_advance", pos_advance_kernel, dim3((B + 63) / 64), dim3(64), 0, (int32_t*)pos, B);
}

// ------------------------------------------------------------------------------------------------ seeded fills
// word(seed, c): splitmix64 finaliser of seed + (c+1)*golden.  Integer-only, so host and device agree bit for bit.
__device__ __forceinline__ unsigned long long synth_word(unsigned long long seed, unsigned long long c) {
  unsigned long long z = seed + (c + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ uint32_t synth_sum16(unsigned long long w) {
  return (uint32_t)(w & 0xFFFF) + (uint32_t)((w >> 16) & 0xFFFF) + (uint32_t)((w >> 32) & 0xFFFF) + (uint32_t)(w >> 48);
}

// Irwin-Hall normal: sum of twelve uniform 16-bit integers, centred and scaled by one fp32 multiply.
__global__ void fill_normal_f16_kernel(__half* __restrict__ dst, unsigned long long seed, unsigned long long first,
                                       unsigned long long n, float c) {
  for (unsigned long long j = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; j < n;
       j += (unsigned long long)gridDim.x * blockDim.x) {
    unsigned long long i = first + j;
    int S = (int)(synth_sum16(synth_word(seed, 3 * i)) + synth_sum16(synth_word(seed, 3 * i + 1)) +
                  synth_sum16(synth_word(seed, 3 * i + 2)));
    dst[j] = __float2half_rn(__fmul_rn((float)(S - 393210), c));
  }
}
__global__ void fill_uniform_i8_kernel(int8_t* __restrict__ dst, unsigned long long seed, unsigned long long first,
                                       unsigned long long n) {
  for (unsigned long long j = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; j < n;
       j += (unsigned long long)gridDim.x * blockDim.x)
    dst[j] = (int8_t)((int)(((synth_word(seed, first + j) >> 32) * 255ull) >> 32) - 127);
}
__global__ void fill_scale_f16_kernel(__half* __restrict__ dst, unsigned long long seed, unsigned long long first,
                                      unsigned long long n, float base) {
  for (unsigned long long j = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; j < n;
       j += (unsigned long long)gridDim.x * blockDim.x) {
    float u = __fadd_rn(0.5f, __fmul_rn((float)(synth_word(seed, first + j) >> 40), 5.9604644775390625e-08f));
    dst[j] = __float2half_rn(__fmul_rn(u, base));
  }
}
__global__ void fill_const_f16_kernel(__half* __restrict__ dst, unsigned long long n, __half v) {
  for (unsigned long long j = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; j < n;
       j += (unsigned long long)gridDim.x * blockDim.x)
    dst[j] = v;
}

static inline int fill_blocks(jg_dev* dev, uint64_t n) {
  uint64_t b = (n + 255) / 256;
  uint64_t cap = (uint64_t)dev->sm_count * 16;
  return (int)(b < cap ? b : cap);
}

JG_API int jg_fill_normal_f16(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t first, uint64_t n, float std) {
  JG_ENTER(dev);
  JG_REQUIRE(n > 0 && jg_aligned(dst, 2), "fill_normal_f16: bad arguments");
  jg_mark_fresh(dev, dst, n * 2);
  fill_normal_f16_kernel<<<fill_blocks(dev, n), 256, 0, dev->stream>>>((__half*)dst, seed, first, n, std / 65536.0f);
  return jg_after_launch(dev, "fill_normal_f16");
}
JG_API int jg_fill_uniform_i8(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t first, uint64_t n) {
  JG_ENTER(dev);
  JG_REQUIRE(n > 0 && dst != 0, "fill_uniform_i8: bad arguments");
  jg_mark_fresh(dev, dst, n);
  fill_uniform_i8_kernel<<<fill_blocks(dev, n), 256, 0, dev->stream>>>((int8_t*)dst, seed, first, n);
  return jg_after_launch(dev, "fill_uniform_i8");
}
JG_API int jg_fill_scale_f16(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t first, uint64_t n, float base) {
  JG_ENTER(dev);
  JG_REQUIRE(n > 0 && jg_aligned(dst, 2), "fill_scale_f16: bad arguments");
  jg_mark_fresh(dev, dst, n * 2);
  fill_scale_f16_kernel<<<fill_blocks(dev, n), 256, 0, dev->stream>>>((__half*)dst, seed, first, n, base);
  return jg_after_launch(dev, "fill_scale_f16");
}
JG_API int jg_fill_const_f16(jg_dev* dev, uint64_t dst, uint64_t n, float value) {
  JG_ENTER(dev);
  JG_REQUIRE(n > 0 && jg_aligned(dst, 2), "fill_const_f16: bad arguments");
  jg_mark_fresh(dev, dst, n * 2);
  fill_const_f16_kernel<<<fill_blocks(dev, n), 256, 0, dev->stream>>>((__half*)dst, n, __float2half_rn(value));
  return jg_after_launch(dev, "fill_const_f16");
}

// ------------------------------------------------------------------------------------------------ int8 -> fp16 weights
// The dequantised matrix of Int8Linear.call (jsgrad/models/llama3.ts:35: weight.cast(half) * scale, one fp16 rounding per
// element), materialised once so that a many-row projection can run on the fp16 tensor-core kernel — what the reference
// graph itself does when a call has more than one row.
__global__ void dequant_i8_f16_kernel(__half* __restrict__ dst, const int8_t* __restrict__ w, const __half* __restrict__ scale,
                                      long long n16, int k16) {
  pdl_launch();
  pdl_wait();
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < n16; c += (long long)gridDim.x * blockDim.x) {
    const long long row = c / k16;
    const uint4 raw = ld_stream_128(reinterpret_cast<const uint4*>(w) + c);
    const __half s = scale[row];
    const int8_t* q = reinterpret_cast<const int8_t*>(&raw);
    __align__(16) __half o[16];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i] = hmul1(__int2half_rn((int)q[i]), s);
    reinterpret_cast<uint4*>(dst)[2 * c] = *reinterpret_cast<uint4*>(&o[0]);
    reinterpret_cast<uint4*>(dst)[2 * c + 1] = *reinterpret_cast<uint4*>(&o[8]);
  }
}

JG_API int jg_dequant_i8_f16(jg_dev* dev, uint64_t dst, uint64_t w, uint64_t scale, int64_t N, int64_t K) {
  JG_ENTER(dev);
  JG_REQUIRE(N > 0 && K > 0 && K % 16 == 0, "dequant_i8_f16: bad shape N=%lld K=%lld (K must be a multiple of 16)", (long long)N, (long long)K);
  JG_REQUIRE(jg_aligned(dst, 16) && jg_aligned(w, 16) && jg_aligned(scale, 2), "dequant_i8_f16: null or misaligned pointer");
  const long long n16 = N * K / 16;
  jg_mark_fresh(dev, dst, (uint64_t)N * K * 2);
  long long blocks = (n16 + 255) / 256;
  if (blocks > (long long)dev->sm_count * 16) blocks = (long long)dev->sm_count * 16;
  return jg_launch(dev, "dequant_i8_f16", dequant_i8_f16_kernel, dim3((unsigned)blocks), dim3(256), 0, (__half*)dst,
                   (const int8_t*)w, (const __half*)scale, n16, (int)(K / 16));
}

// NF4Linear's dequantised matrix (jsgrad/models/llama3.ts:88-94): element i of the flattened [out][in] matrix is
// half(CODE[code_i] * scale[i / block]) with code_2j in the high nibble of byte j and code_2j+1 in the low one, the 16
// code values rounded to fp16 first (:81).  One thread turns 16 packed bytes into 32 halves.
__constant__ float c_nf4_code[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                     -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                     0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
                                     0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
                                     0.7229568362236023f, 1.0f};
__global__ void dequant_nf4_f16_kernel(__half* __restrict__ dst, const uint8_t* __restrict__ w, const __half* __restrict__ scale,
                                       long long n32, int block) {
  __shared__ __half code[16];
  if (threadIdx.x < 16) code[threadIdx.x] = __float2half_rn(c_nf4_code[threadIdx.x]);
  pdl_launch();
  pdl_wait();
  __syncthreads();
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < n32; c += (long long)gridDim.x * blockDim.x) {
    const uint4 raw = ld_stream_128(reinterpret_cast<const uint4*>(w) + c);
    const uint8_t* q = reinterpret_cast<const uint8_t*>(&raw);
    __align__(16) __half o[32];
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const long long e = c * 32 + 2 * i;  // blocks hold an even number of elements: both nibbles share a scale
      const __half s = scale[e / block];
      o[2 * i] = hmul1(code[q[i] >> 4], s);
      o[2 * i + 1] = hmul1(code[q[i] & 15], s);
    }
#pragma unroll
    for (int v = 0; v < 4; v++) reinterpret_cast<uint4*>(dst)[4 * c + v] = *reinterpret_cast<uint4*>(&o[8 * v]);
  }
}

JG_API int jg_dequant_nf4_f16(jg_dev* dev, uint64_t dst, uint64_t w, uint64_t scale, int64_t n, int32_t block) {
  JG_ENTER(dev);
  JG_REQUIRE(n > 0 && n % 32 == 0 && block >= 2 && block % 2 == 0 && n % block == 0,
             "dequant_nf4_f16: n=%lld must be a multiple of 32 and of the (even) block size %d", (long long)n, block);
  JG_REQUIRE(jg_aligned(dst, 16) && jg_aligned(w, 16) && jg_aligned(scale, 2), "dequant_nf4_f16: null or misaligned pointer");
  const long long n32 = n / 32;
  jg_mark_fresh(dev, dst, (uint64_t)n * 2);
  long long blocks = (n32 + 255) / 256;
  if (blocks > (long long)dev->sm_count * 16) blocks = (long long)dev->sm_count * 16;
  return jg_launch(dev, "dequant_nf4_f16", dequant_nf4_f16_kernel, dim3((unsigned)blocks), dim3(256), 0, (__half*)dst,
                   (const uint8_t*)w, (const __half*)scale, n32, (int)block);
}

// ------------------------------------------------------------------------------------------------ tensor-parallel helpers
// h <- h + half(p): the residual add of TransformerBlock.call (jsgrad/models/llama.ts:125-126) applied to the fp32 sum
// of a row-parallel projection after its all-reduce: one rounding of the full sum to fp16, then the fp16 add, exactly
// as on a single device.
__global__ void residual_add_f32_kernel(__half* __restrict__ h, const float* __restrict__ p, long long n4) {
  pdl_launch();
  pdl_wait();
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < n4; c += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(p)[c];
    uint2 raw = reinterpret_cast<uint2*>(h)[c];
    __half* hh = reinterpret_cast<__half*>(&raw);
    hh[0] = hadd1(hh[0], __float2half_rn(v.x));
    hh[1] = hadd1(hh[1], __float2half_rn(v.y));
    hh[2] = hadd1(hh[2], __float2half_rn(v.z));
    hh[3] = hadd1(hh[3], __float2half_rn(v.w));
    reinterpret_cast<uint2*>(h)[c] = raw;
  }
}

JG_API int jg_residual_add_f32(jg_dev* dev, uint64_t h, uint64_t p32, int64_t n) {
  JG_ENTER(dev);
  JG_REQUIRE(n > 0 && n % 4 == 0, "residual_add_f32: element count %lld must be a positive multiple of 4", (long long)n);
  JG_REQUIRE(jg_aligned(h, 8) && jg_aligned(p32, 16), "residual_add_f32: null or misaligned pointer");
  const long long n4 = n / 4;
  int blocks = (int)((n4 + 255) / 256);
  if (blocks > dev->sm_count * 4) blocks = dev->sm_count * 4;
  return jg_launch(dev, "residual_add_f32", residual_add_f32_kernel, dim3(blocks), dim3(256), 0, (__half*)h, (const float*)p32, n4);
}

// Seeded normal fill of a [rows][cols] window of a [*][full_cols] tensor starting at (row0, col0): element (r, c) takes
// generator index (row0 + r) * full_cols + col0 + c, so a shard holds exactly the values the whole tensor would.
__global__ void fill_normal_f16_2d_kernel(__half* __restrict__ dst, unsigned long long seed, unsigned long long rows,
                                          unsigned long long cols, unsigned long long full_cols, unsigned long long row0,
                                          unsigned long long col0, float c) {
  const unsigned long long n = rows * cols;
  for (unsigned long long j = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; j < n;
       j += (unsigned long long)gridDim.x * blockDim.x) {
    const unsigned long long r = j / cols, cc = j % cols;
    const unsigned long long i = (row0 + r) * full_cols + col0 + cc;
    int S = (int)(synth_sum16(synth_word(seed, 3 * i)) + synth_sum16(synth_word(seed, 3 * i + 1)) +
                  synth_sum16(synth_word(seed, 3 * i + 2)));
    dst[j] = __float2half_rn(__fmul_rn((float)(S - 393210), c));
  }
}

// The int8 counterpart: element (r, c) of the window takes generator index (row0 + r) * full_cols + col0 + c.
__global__ void fill_uniform_i8_2d_kernel(int8_t* __restrict__ dst, unsigned long long seed, unsigned long long rows,
                                          unsigned long long cols, unsigned long long full_cols, unsigned long long row0,
                                          unsigned long long col0) {
  const unsigned long long n = rows * cols;
  for (unsigned long long j = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; j < n;
       j += (unsigned long long)gridDim.x * blockDim.x) {
    const unsigned long long r = j / cols, cc = j % cols;
    const unsigned long long i = (row0 + r) * full_cols + col0 + cc;
    dst[j] = (int8_t)((int)(((synth_word(seed, i) >> 32) * 255ull) >> 32) - 127);
  }
}

JG_API int jg_fill_uniform_i8_2d(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t rows, uint64_t cols, uint64_t full_cols,
                                 uint64_t row0, uint64_t col0) {
  JG_ENTER(dev);
  JG_REQUIRE(rows > 0 && cols > 0 && col0 + cols <= full_cols && dst != 0, "fill_uniform_i8_2d: bad arguments");
  jg_mark_fresh(dev, dst, rows * cols);
  fill_uniform_i8_2d_kernel<<<fill_blocks(dev, rows * cols), 256, 0, dev->stream>>>((int8_t*)dst, seed, rows, cols, full_cols, row0, col0);
  return jg_after_launch(dev, "fill_uniform_i8_2d");
}

JG_API int jg_fill_normal_f16_2d(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t rows, uint64_t cols, uint64_t full_cols,
                                 uint64_t row0, uint64_t col0, float std) {
  JG_ENTER(dev);
  JG_REQUIRE(rows > 0 && cols > 0 && col0 + cols <= full_cols && jg_aligned(dst, 2), "fill_normal_f16_2d: bad arguments");
  jg_mark_fresh(dev, dst, rows * cols * 2);
  fill_normal_f16_2d_kernel<<<fill_blocks(dev, rows * cols), 256, 0, dev->stream>>>((__half*)dst, seed, rows, cols, full_cols,
                                                                                   row0, col0, std / 65536.0f);
  return jg_after_launch(dev, "fill_normal_f16_2d");
}
