/*
 * llama_oracle.c — CPU restatement of jsgrad's Llama-3 forward (prefill + KV-cached greedy decode).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is compared against; it is never
 * linked into, imported by, or called from the shipped library.  Only the test-suite, the smoke check and the
 * CPU-baseline / reference legs of the benchmark may load it.
 *
 * PARITY UNPINNED: the reference repository holds no golden vectors, known-answer tests or fixtures for this
 * path (its tests diff against an un-vendored Python tinygrad submodule), and the reference cannot be executed
 * where this is built (no JS runtime, no clang).  The arithmetic below is therefore restated from the
 * reference's *source*; every function cites the lines it follows (paths are relative to the reference
 * project root).
 *
 * Numeric conventions (each one is the reference's IR semantics, as executed op by op):
 *  - a reduction (dot product, attention scores, p.v, sum of squares) forms the exact fp32 product of its fp16
 *    operands and accumulates in fp32 in strictly ascending index order, then rounds once
 *    (jsgrad/tensor.ts:2593-2605 `dot`, :1967-1970 `sum`, jsgrad/dtype.ts:243-248 `sum_acc_dtype`;
 *    ascending sequential order: jsgrad/codegen/lowerer.ts:130-146);
 *  - every elementwise op whose IR dtype is fp16 rounds its result to fp16 once (jsgrad/ops.ts:757-761 `exec_alu`
 *    with jsgrad/dtype.ts:250-265 `truncate`);
 *  - exp2 and sin are the in-tree polynomial versions (jsgrad/ops.ts:1625-1673), because the CLANG renderer has
 *    no native EXP2/SIN (jsgrad/renderer/cstyle.ts:214-217); sqrt is sqrtf, reciprocal is 1/x;
 *  - no FMA contraction, no fast-math (build with -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 h16;

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------------------
 * helpers: one rounding per fp16 elementwise op
 * ---------------------------------------------------------------------------------------------------------- */
static inline h16 hmul(h16 a, h16 b) { return (h16)((float)a * (float)b); } /* product exact in fp32 -> 1 rounding */
static inline h16 hadd(h16 a, h16 b) { return (h16)((float)a + (float)b); } /* sum exact in fp32 -> 1 rounding */
static inline h16 hsub(h16 a, h16 b) { return (h16)((float)a - (float)b); }
static inline h16 hrecip(h16 a) { return (h16)(1.0f / (float)a); } /* fp32 quotient of an fp16 is within the
                                                                       double-rounding-safe range (24 >= 2*11+2) */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t h2u(h16 h) { uint16_t u; memcpy(&u, &h, 2); return u; }
static inline h16 u2h(uint16_t u) { h16 h; memcpy(&h, &u, 2); return h; }

/* ------------------------------------------------------------------------------------------------------------
 * xexp2, fp32 branch — jsgrad/ops.ts:1650-1673 (`xexp2`), :1465-1468 (`rintk`), :1471-1474 (`pow2if`),
 * :1491-1494 (`ldexp2k`), jsgrad/helpers/helpers.ts:810 (`polyN`, Horner from the highest coefficient).
 * ---------------------------------------------------------------------------------------------------------- */
static inline float pow2if_f32(int32_t q) { return u2f((uint32_t)(q + 127) << 23); }

ORC_API float orc_xexp2_f32(float d) {
  float x = (d != INFINITY) ? ((d != d) ? 0.0f : ((d != -INFINITY) ? d : 0.0f)) : 0.0f; /* _lazy_map_numbers */
  int32_t q = (int32_t)(x + (x < 0.0f ? -0.5f : 0.5f));                                   /* rintk: trunc cast */
  float s = x - (float)q;
  static const float c[7] = {0.1535920892e-3f, 0.1339262701e-2f, 0.9618384764e-2f, 0.5550347269e-1f,
                             0.2402264476e+0f, 0.6931471825e+0f, 1.0f};
  float u = c[0]; /* polyN: ((0*x)+c0) folds to c0 */
  for (int i = 1; i < 7; i++) u = u * s + c[i];
  int32_t q1 = q / 2; /* shr(e,1) is idiv by 2: C truncation */
  u = (u * pow2if_f32(q1)) * pow2if_f32(q - q1);
  if (d >= 128.0f) u = INFINITY;
  if (d < -150.0f) u = 0.0f;
  if (d != d) u = NAN;
  return u;
}

/* xexp2, fp16 branch: same graph with every op in fp16 (int16 rintk, bounds 23 / -22). */
ORC_API uint16_t orc_xexp2_f16(uint16_t dbits) {
  h16 d = u2h(dbits);
  float df = (float)d;
  h16 x = (df != INFINITY) ? ((df != df) ? (h16)0.0f : ((df != -INFINITY) ? d : (h16)0.0f)) : (h16)0.0f;
  h16 xr = hadd(x, ((float)x < 0.0f) ? (h16)-0.5f : (h16)0.5f);
  float xrf = (float)xr;
  if (xrf > 32767.0f) xrf = 32767.0f; /* the cast of an out-of-range value is undefined in C; the result is */
  if (xrf < -32768.0f) xrf = -32768.0f; /* overwritten by the bound checks below in that range anyway        */
  int16_t q = (int16_t)xrf;
  h16 s = hsub(x, (h16)(float)q);
  static const float c[7] = {0.1535920892e-3f, 0.1339262701e-2f, 0.9618384764e-2f, 0.5550347269e-1f,
                             0.2402264476e+0f, 0.6931471825e+0f, 1.0f};
  h16 u = (h16)c[0];
  for (int i = 1; i < 7; i++) u = hadd(hmul(u, s), (h16)c[i]);
  int16_t q1 = (int16_t)(q / 2);
  int16_t q2 = (int16_t)(q - q1);
  /* pow2if on int16: shl(q + 15, 10) bit-cast to half (jsgrad/ops.ts:1471-1474) */
  h16 p1 = u2h((uint16_t)((int16_t)(q1 + 15) * 1024));
  h16 p2 = u2h((uint16_t)((int16_t)(q2 + 15) * 1024));
  u = hmul(hmul(u, p1), p2);
  if (df >= 23.0f) u = (h16)INFINITY;
  if (df < -22.0f) u = (h16)0.0f;
  if (df != df) u = (h16)NAN;
  return h2u(u);
}

/* ------------------------------------------------------------------------------------------------------------
 * xsin, fp32 — jsgrad/ops.ts:1625-1644 (`xsin`, fast=false, switch_over=30), :1564-1594 (`cody_waite_reduction`,
 * fp32 branch), :1513-1558 (`payne_hanek_reduction`), :1596-1620 (`sin_poly*`), :1496-1508 (`frexp`).
 * ---------------------------------------------------------------------------------------------------------- */
static inline float sin_poly(float d) {
  static const float c[5] = {2.6083159809786593541503e-06f, -0.0001981069071916863322258f,
                             0.00833307858556509017944336f, -0.166666597127914428710938f, 1.0f};
  float d2 = d * d;
  float u = c[0];
  for (int i = 1; i < 5; i++) u = u * d2 + c[i];
  return d * u;
}

static void cody_waite_f32(float d, float* r, int32_t* q) {
  const float m_1_pi = 0.318309886183790671537767526745028724f;
  float t = d * m_1_pi;
  int32_t quad = (int32_t)(t + (t < 0.0f ? -0.5f : 0.5f));
  float qf = (float)quad;
  float v = qf * -3.1414794921875f + d;
  v = qf * -0.00011315941810607910156f + v;
  v = qf * -1.9841872589410058936e-09f + v;
  v = qf * -1.2154201256553420762e-10f + v;
  *r = v;
  *q = quad;
}

static void payne_hanek_f32(float d, float* r, int32_t* q) {
  static const uint32_t two_over_pi_f[7] = {0x00000000u, 0x28be60dbu, 0x9391054au, 0x7f09d5f4u,
                                            0x7d4d3770u, 0x36d8a566u, 0x4f10e410u};
  uint32_t bits = f2u(d);
  uint32_t exponent = (bits >> 23) & 255u;
  float f = u2f((bits & 0x807FFFFFu) | 0x3F000000u);
  int32_t e = (int32_t)exponent - 127 + 1;
  uint64_t ia = (uint64_t)(f * 4.294967296e9f);
  uint64_t i = ((uint64_t)(int64_t)e) >> 5;
  e = e & 31;
  int32_t offset = 32 - e;
  uint32_t a[4];
  for (int n = 0; n < 4; n++) { /* `_take`: two_over_pi_f[i + n]; the last table entry closes the chain */
    uint64_t idx = i + (uint64_t)n;
    a[n] = two_over_pi_f[idx < 6 ? idx : 6];
  }
#define SHL_LAZY(x, y) ((uint32_t)((uint64_t)(x) * (uint64_t)pow2if_f32(y)))
#define SHR_LAZY(x, y) ((uint32_t)((uint64_t)(x) / (uint64_t)pow2if_f32(y)))
  uint32_t hi = SHL_LAZY(a[0], e) | SHR_LAZY(a[1], offset);
  uint32_t mi = SHL_LAZY(a[1], e) | SHR_LAZY(a[2], offset);
  uint32_t lo = SHL_LAZY(a[2], e) | SHR_LAZY(a[3], offset);
#undef SHL_LAZY
#undef SHR_LAZY
  uint64_t p = ((ia * (uint64_t)hi) << 32) + (ia * (uint64_t)mi) + ((ia * (uint64_t)lo) >> 32);
  int32_t quad = (int32_t)(p >> 62);
  p &= 0x3fffffffffffffffull;
  float rr = (float)p * 3.4061215800865545e-19f;
  /* the source tests the frexp mantissa (always in [0.5,1)) against 0.5, as written at ops.ts:1557 */
  if (f < 0.5f) { *r = rr; *q = quad; }
  else { *r = rr - (float)(M_PI / 2); *q = quad + 1; }
}

ORC_API float orc_xsin_f32(float d) {
  float x = (d != INFINITY) ? ((d != d) ? 0.0f : ((d != -INFINITY) ? d : 0.0f)) : 0.0f;
  float x_sign = (x != 0.0f) ? ((x < 0.0f) ? -1.0f : 1.0f) : 0.0f;
  float x_abs = x * x_sign;
  float r, rs;
  int32_t q, qs;
  float result;
  if (x_abs < 30.0f) {
    cody_waite_f32(x_abs, &rs, &qs);
    float v = sin_poly(rs);
    result = v * ((qs & 1) ? -1.0f : 1.0f);
  } else {
    payne_hanek_f32(x_abs, &r, &q);
    float v = sin_poly(r + ((q & 1) ? (float)(M_PI / 2) : 0.0f));
    result = v * ((q & 2) ? -1.0f : 1.0f);
  }
  result = result * x_sign;
  if (d == INFINITY || d == -INFINITY || d != d) result = NAN;
  return result;
}

/* ------------------------------------------------------------------------------------------------------------
 * precompute_freqs_cis — jsgrad/models/llama.ts:10-14, cast to fp16 at :205.
 *   freqs = 1 / theta^(arange(0,hd,2)/hd) with `pow(theta, reverse)` = exp(x*ln theta) (jsgrad/tensor.ts:3709)
 *   and exp(y) = exp2(y * 1/ln2) (jsgrad/tensor.ts:147-151); the chained constant multiplies fold into one
 *   (jsgrad/ops.ts:1363).  cos(x) = sin(pi/2 - x) (jsgrad/tensor.ts:2964-2966).
 * out: [end][hd/2][2] fp16 = (cos, sin).
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API void orc_freqs_cis(int head_dim, int end, double theta, uint16_t* out) {
  int half = head_dim / 2;
  float recip_dim = (float)(1.0 / (double)head_dim);
  float c = (float)((double)recip_dim * log(theta) * (1.0 / log(2.0)));
  float* freq = (float*)malloc(sizeof(float) * (size_t)half);
  for (int i = 0; i < half; i++) {
    float p = orc_xexp2_f32((float)(2 * i) * c);
    freq[i] = 1.0f / p;
  }
  const float half_pi = (float)(M_PI / 2);
#pragma omp parallel for schedule(static)
  for (int t = 0; t < end; t++) {
    for (int i = 0; i < half; i++) {
      float ang = (float)t * freq[i];
      float co = orc_xsin_f32(half_pi - ang);
      float si = orc_xsin_f32(ang);
      out[((size_t)t * half + i) * 2 + 0] = h2u((h16)co);
      out[((size_t)t * half + i) * 2 + 1] = h2u((h16)si);
    }
  }
  free(freq);
}

/* ------------------------------------------------------------------------------------------------------------
 * RMSNorm — jsgrad/nn/index.ts:586-588: `_norm(x.float()).cast(half).mul(weight)`,
 *   _norm(x) = x * sqrt(1/(mean(x^2)+eps)); mean = fp32 sum * (1/d) (jsgrad/tensor.ts:2113-2117,3576-3579),
 *   rsqrt = reciprocal().sqrt() (jsgrad/tensor.ts:2944-2946).
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API void orc_rmsnorm(const uint16_t* x_, const uint16_t* w_, uint16_t* y_, int rows, int d, float eps) {
  const h16* x = (const h16*)x_;
  const h16* w = (const h16*)w_;
  h16* y = (h16*)y_;
  const float recip_d = (float)(1.0 / (double)d);
  for (int r = 0; r < rows; r++) {
    const h16* xr = x + (size_t)r * d;
    float ss = 0.0f;
    for (int k = 0; k < d; k++) { float v = (float)xr[k]; ss = ss + v * v; }
    float m = ss * recip_d;
    float rs = sqrtf(1.0f / (m + eps));
    for (int k = 0; k < d; k++) y[(size_t)r * d + k] = hmul((h16)((float)xr[k] * rs), w[k]);
  }
}

/* ------------------------------------------------------------------------------------------------------------
 * Linear — jsgrad/nn/index.ts:411 -> jsgrad/tensor.ts:3800-3803,2593-2605: y[m,o] = half(sum_k x[m,k]*W[o,k]),
 * fp32 ascending-k accumulation.  Rows are processed in blocks of 8 independent accumulators so that the
 * sequential adds of different outputs overlap; the order of additions inside each output is unchanged.
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API void orc_linear_f16(const uint16_t* x_, const uint16_t* w_, uint16_t* y_, int M, int N, int K) {
  const h16* x = (const h16*)x_;
  const h16* w = (const h16*)w_;
  h16* y = (h16*)y_;
  for (int m = 0; m < M; m++) {
    const h16* xm = x + (size_t)m * K;
#pragma omp parallel for schedule(static)
    for (int ob = 0; ob < (N + 7) / 8; ob++) {
      int o0 = ob * 8;
      int nr = N - o0 < 8 ? N - o0 : 8;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      const h16* wr[8];
      for (int j = 0; j < 8; j++) wr[j] = w + (size_t)(o0 + (j < nr ? j : 0)) * K;
      for (int k = 0; k < K; k++) {
        float xv = (float)xm[k];
        for (int j = 0; j < 8; j++) acc[j] = acc[j] + xv * (float)wr[j][k];
      }
      for (int j = 0; j < nr; j++) y[(size_t)m * N + o0 + j] = (h16)acc[j];
    }
  }
}

/* Int8Linear — jsgrad/models/llama3.ts:35: x.dot(W.cast(half).T * scale): the dequantised weight
 * half(Wq[o,k]) * s[o] is an fp16 elementwise product (one rounding), then the fp16 dot above. */
ORC_API void orc_linear_w8(const uint16_t* x_, const int8_t* wq, const uint16_t* s_, uint16_t* y_, int M, int N, int K) {
  const h16* x = (const h16*)x_;
  const h16* s = (const h16*)s_;
  h16* y = (h16*)y_;
  for (int m = 0; m < M; m++) {
    const h16* xm = x + (size_t)m * K;
#pragma omp parallel for schedule(static)
    for (int ob = 0; ob < (N + 7) / 8; ob++) {
      int o0 = ob * 8;
      int nr = N - o0 < 8 ? N - o0 : 8;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      const int8_t* wr[8];
      h16 sc[8];
      for (int j = 0; j < 8; j++) { int o = o0 + (j < nr ? j : 0); wr[j] = wq + (size_t)o * K; sc[j] = s[o]; }
      for (int k = 0; k < K; k++) {
        float xv = (float)xm[k];
        for (int j = 0; j < 8; j++) acc[j] = acc[j] + xv * (float)hmul((h16)(float)wr[j][k], sc[j]);
      }
      for (int j = 0; j < nr; j++) y[(size_t)m * N + o0 + j] = (h16)acc[j];
    }
  }
}

/* Int8Linear.quantize — jsgrad/models/llama3.ts:42-45: scale = max|row|/127 in fp16, Wq = round(W/scale).
 * `div` is x * reciprocal(y) in fp16 (jsgrad/tensor.ts:3576-3579); `round` (jsgrad/tensor.ts:3054-3057) picks
 * ceil(x-0.5) or floor(x+0.5) by the parity of trunc(x), which is round-half-to-even. */
ORC_API void orc_quantize_w8(const uint16_t* w_, int8_t* wq, uint16_t* s_, int N, int K) {
  const h16* w = (const h16*)w_;
  h16* s = (h16*)s_;
#pragma omp parallel for schedule(static)
  for (int o = 0; o < N; o++) {
    float mx = 0.0f;
    for (int k = 0; k < K; k++) { float a = fabsf((float)w[(size_t)o * K + k]); if (a > mx) mx = a; }
    h16 sc = hmul((h16)mx, hrecip((h16)127.0f));
    h16 rsc = hrecip(sc);
    s[o] = sc;
    for (int k = 0; k < K; k++) {
      h16 v = hmul(w[(size_t)o * K + k], rsc);
      float r = nearbyintf((float)v); /* default rounding mode: ties to even */
      if (r > 127.0f) r = 127.0f;
      if (r < -128.0f) r = -128.0f;
      wq[(size_t)o * K + k] = (int8_t)r;
    }
  }
}

/* NF4Linear — jsgrad/models/llama3.ts:79-117.  The 16 code values are rounded to fp16 (:81); a weight is
 * half(CODE[c] * scale) with one fp16 scale per block of `block` consecutive elements of the flattened matrix (:92-93);
 * the packed byte holds element 2i in its high nibble and element 2i+1 in its low one (:91,:105).
 * quantize (:96-106): scale = max|block| (fp16), code = argmin_c |half(half(v * half(1/scale)) - CODE[c])|, lowest index
 * among equals. */
static const float ORC_NF4_CODE[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                        -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                        0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
                                        0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
                                        0.7229568362236023f, 1.0f};
ORC_API void orc_nf4_dequant(const uint8_t* packed, const uint16_t* s_, uint16_t* out_, int64_t n, int block) {
  const h16* s = (const h16*)s_;
  h16* out = (h16*)out_;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    const uint8_t b = packed[i / 2];
    const int c = (i & 1) ? (b & 15) : (b >> 4);
    out[i] = hmul((h16)ORC_NF4_CODE[c], s[i / block]);
  }
}
ORC_API void orc_nf4_quantize(const uint16_t* w_, uint8_t* packed, uint16_t* s_, int64_t n, int block) {
  const h16* w = (const h16*)w_;
  h16* s = (h16*)s_;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < n / block; g++) {
    float mx = 0.0f;
    for (int j = 0; j < block; j++) { float a = fabsf((float)w[g * block + j]); if (a > mx) mx = a; }
    const h16 sc = (h16)mx, rsc = hrecip(sc);
    s[g] = sc;
    for (int j = 0; j < block; j += 2) {
      int code[2];
      for (int e = 0; e < 2; e++) {
        const h16 v = hmul(w[g * block + j + e], rsc);
        int best = 0;
        float bd = INFINITY;
        for (int c = 0; c < 16; c++) {
          const float dist = fabsf((float)hsub(v, (h16)ORC_NF4_CODE[c]));
          if (dist < bd) { bd = dist; best = c; }
        }
        code[e] = best;
      }
      packed[(g * block + j) / 2] = (uint8_t)(code[0] * 16 + code[1]);
    }
  }
}

/* ------------------------------------------------------------------------------------------------------------
 * Embedding — jsgrad/nn/index.ts:607-619 (one-hot sum == row gather, exact);
 * Int8Embedding — jsgrad/models/llama3.ts:71-77: row = half(Wq[v,:]) * scale[v] (fp16 product).
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API void orc_embed_f16(const int32_t* idx, const uint16_t* w, uint16_t* out, int n, int d) {
  for (int i = 0; i < n; i++) memcpy(out + (size_t)i * d, w + (size_t)idx[i] * d, (size_t)d * 2);
}
ORC_API void orc_embed_w8(const int32_t* idx, const int8_t* wq, const uint16_t* s_, uint16_t* out_, int n, int d) {
  const h16* s = (const h16*)s_;
  h16* out = (h16*)out_;
  for (int i = 0; i < n; i++)
    for (int k = 0; k < d; k++) out[(size_t)i * d + k] = hmul((h16)(float)wq[(size_t)idx[i] * d + k], s[idx[i]]);
}

/* ------------------------------------------------------------------------------------------------------------
 * apply_rotary_emb / complex_mult — jsgrad/models/llama.ts:17-32: interleaved pairs (x[2i], x[2i+1]),
 *   ro = a*c - b*d, co = a*d + b*c, every op fp16.   x: [rows][n_heads][hd], in place; pos[r] indexes the table.
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API void orc_rope(uint16_t* x_, const uint16_t* table_, const int32_t* pos, int rows, int n_heads, int hd) {
  h16* x = (h16*)x_;
  const h16* table = (const h16*)table_;
  int half = hd / 2;
  for (int r = 0; r < rows; r++)
    for (int h = 0; h < n_heads; h++) {
      h16* v = x + ((size_t)r * n_heads + h) * hd;
      const h16* t = table + (size_t)pos[r] * half * 2;
      for (int i = 0; i < half; i++) {
        h16 a = v[2 * i], b = v[2 * i + 1], c = t[2 * i], d = t[2 * i + 1];
        v[2 * i] = hsub(hmul(a, c), hmul(b, d));
        v[2 * i + 1] = hadd(hmul(a, d), hmul(b, c));
      }
    }
}

/* ------------------------------------------------------------------------------------------------------------
 * scaled_dot_product_attention for one query row against T cached positions —
 * jsgrad/tensor.ts:3920-3934 (fp32 score accumulate, multiply by 1/sqrt(hd), additive mask),
 * :2186-2214 (softmax: subtract max, exp = exp2(x*1/ln2), divide by the sum = multiply by reciprocal),
 * cast to fp16, then p.v with fp32 accumulation; repeat_kv head mapping jsgrad/models/llama.ts:34-39.
 * k, v: [T][n_kv][hd] (one batch row of the cache); q: [H][hd]; out: [H][hd]; positions >= t_visible are
 * masked (-inf) exactly like the additive triu mask built at jsgrad/models/llama.ts:208.
 * ---------------------------------------------------------------------------------------------------------- */
static void attention_row(const h16* q, const h16* k, const h16* v, h16* out, int H, int G, int hd, int T,
                          int t_visible, float* sc) {
  const int n_rep = H / G;
  const float scale = (float)(1.0 / (double)(float)sqrt((double)hd));
  const float log2e = (float)(1.0 / log(2.0));
  for (int h = 0; h < H; h++) {
    int g = h / n_rep;
    const h16* qh = q + (size_t)h * hd;
    float mx = -INFINITY;
    for (int t = 0; t < T; t++) {
      const h16* kt = k + ((size_t)t * G + g) * hd;
      float acc = 0.0f;
      for (int i = 0; i < hd; i++) acc = acc + (float)qh[i] * (float)kt[i];
      float s = acc * scale;
      if (t >= t_visible) s = s + -INFINITY;
      sc[t] = s;
      if (s > mx) mx = s;
    }
    float sum = 0.0f;
    for (int t = 0; t < T; t++) {
      float e = orc_xexp2_f32((sc[t] - mx) * log2e);
      sc[t] = e;
      sum = sum + e;
    }
    float rsum = 1.0f / sum;
    h16* oh = out + (size_t)h * hd;
    for (int i = 0; i < hd; i++) {
      float acc = 0.0f;
      for (int t = 0; t < T; t++) {
        h16 p = (h16)(sc[t] * rsum);
        acc = acc + (float)p * (float)v[((size_t)t * G + g) * hd + i];
      }
      oh[i] = (h16)acc;
    }
  }
}

/* Stand-alone attention over a contiguous cache: q [B][S][H][hd], k/v [B][Tmax][G][hd], out [B][S][H*hd];
 * query row s of the S new tokens sees positions [0, start_pos + s]. */
ORC_API void orc_attention(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out, int B, int S,
                           int H, int G, int hd, int Tmax, int start_pos) {
  int T = start_pos + S;
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int b = 0; b < B; b++)
    for (int s = 0; s < S; s++) {
      float* sc = (float*)malloc(sizeof(float) * (size_t)T);
      attention_row((const h16*)q + (((size_t)b * S + s) * H) * hd, (const h16*)k + (size_t)b * Tmax * G * hd,
                    (const h16*)v + (size_t)b * Tmax * G * hd, (h16*)out + (((size_t)b * S + s) * H) * hd, H, G, hd,
                    T, S > 1 ? start_pos + s + 1 : T, sc);
      free(sc);
    }
}

/* ------------------------------------------------------------------------------------------------------------
 * SwiGLU elementwise part — jsgrad/models/llama.ts:108-110, jsgrad/tensor.ts:2909-2911,3210-3226:
 *   silu(g) = g * 1/(1 + exp2(g * c)), c = fp16(-1/ln2 * ln2 * 1/ln2) (constants fold, jsgrad/ops.ts:1363),
 *   then * u; every op fp16.
 * ---------------------------------------------------------------------------------------------------------- */
static inline h16 silu_mul(h16 g, h16 u) {
  const h16 c = (h16)(float)((-1.0 / log(2.0)) * log(2.0) * (1.0 / log(2.0)));
  h16 e = u2h(orc_xexp2_f16(h2u(hmul(g, c))));
  h16 sig = hrecip(hadd((h16)1.0f, e));
  return hmul(hmul(g, sig), u);
}
ORC_API void orc_swiglu(const uint16_t* g, const uint16_t* u, uint16_t* out, int n) {
  for (int i = 0; i < n; i++) out[i] = h2u(silu_mul(u2h(g[i]), u2h(u[i])));
}

/* argmax — jsgrad/tensor.ts:2314-2320: lowest index among the maxima. */
ORC_API int32_t orc_argmax_f16(const uint16_t* x_, int n) {
  const h16* x = (const h16*)x_;
  float mx = -INFINITY;
  for (int i = 0; i < n; i++) if ((float)x[i] > mx) mx = (float)x[i];
  for (int i = 0; i < n; i++) if ((float)x[i] == mx) return i;
  return 0;
}

/* ------------------------------------------------------------------------------------------------------------
 * Model: Transformer.forward — jsgrad/models/llama.ts:201-213 with TransformerBlock :124-127,
 * Attention :61-97 (KV cache :78-90), FeedForward :108-110.
 * ---------------------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t dim, n_layers, n_heads, n_kv_heads, hidden, vocab, max_context, max_batch;
  int32_t quant; /* 0: fp16 Linear/Embedding; 1: Int8Linear for attention/ffn weights */
  int32_t quant_embed; /* 1: Int8Embedding and int8 output (quantize_embeds, jsgrad/models/llama3.ts:55-58) */
  float eps;
  double theta;
} orc_config;

enum { ORC_WQ = 0, ORC_WK, ORC_WV, ORC_WO, ORC_W1, ORC_W2, ORC_W3, ORC_ATTN_NORM, ORC_FFN_NORM, ORC_PER_LAYER };
enum { ORC_TOK_EMB = 0, ORC_OUTPUT, ORC_NORM, ORC_GLOBALS };

typedef struct {
  orc_config c;
  const void** layer_w;  /* [L][ORC_PER_LAYER] weight pointers (fp16 or int8), owned by the caller */
  const void** layer_s;  /* [L][ORC_PER_LAYER] fp16 scale pointers for int8 weights */
  const void* glob_w[ORC_GLOBALS];
  const void* glob_s[ORC_GLOBALS];
  h16* cache;  /* [L][2][B][max_context][G][hd] */
  h16* table;  /* [2*max_context][hd/2][2] */
} orc_model;

ORC_API orc_model* orc_model_create(const orc_config* c) {
  orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
  m->c = *c;
  m->layer_w = (const void**)calloc((size_t)c->n_layers * ORC_PER_LAYER, sizeof(void*));
  m->layer_s = (const void**)calloc((size_t)c->n_layers * ORC_PER_LAYER, sizeof(void*));
  int hd = c->dim / c->n_heads;
  size_t cache_n = (size_t)c->n_layers * 2 * c->max_batch * c->max_context * c->n_kv_heads * hd;
  m->cache = (h16*)calloc(cache_n, sizeof(h16));
  m->table = (h16*)malloc(sizeof(h16) * (size_t)2 * c->max_context * hd);
  orc_freqs_cis(hd, 2 * c->max_context, c->theta, (uint16_t*)m->table);
  return m;
}
ORC_API void orc_model_destroy(orc_model* m) {
  if (!m) return;
  free(m->layer_w); free(m->layer_s); free(m->cache); free(m->table); free(m);
}
/* layer < 0 selects the global tensors (which = ORC_TOK_EMB / ORC_OUTPUT / ORC_NORM). Pointers are borrowed. */
ORC_API void orc_model_set_weight(orc_model* m, int layer, int which, const void* w, const void* scale) {
  if (layer < 0) { m->glob_w[which] = w; m->glob_s[which] = scale; }
  else { m->layer_w[(size_t)layer * ORC_PER_LAYER + which] = w; m->layer_s[(size_t)layer * ORC_PER_LAYER + which] = scale; }
}
/* Thread count of the OpenMP loops (the reference's generated C is single-threaded, jsgrad/renderer/cstyle.ts:206; the
 * loops over output rows here are split over threads only to make the checker usable at full width).  A caller that
 * times the checker sets the count explicitly instead of inheriting OMP_NUM_THREADS from a launcher. */
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
ORC_API const uint16_t* orc_model_table(orc_model* m) { return (const uint16_t*)m->table; }
ORC_API uint16_t* orc_model_cache(orc_model* m) { return (uint16_t*)m->cache; }

static void linear_any(const orc_model* m, int layer, int which, const h16* x, h16* y, int M, int N, int K) {
  const void* w = m->layer_w[(size_t)layer * ORC_PER_LAYER + which];
  const void* s = m->layer_s[(size_t)layer * ORC_PER_LAYER + which];
  if (m->c.quant) orc_linear_w8((const uint16_t*)x, (const int8_t*)w, (const uint16_t*)s, (uint16_t*)y, M, N, K);
  else orc_linear_f16((const uint16_t*)x, (const uint16_t*)w, (uint16_t*)y, M, N, K);
}

/* tokens [B][S]; writes the last position's logits (fp16 values widened to fp32, [B][V]) and, per batch row, the
 * greedy token (jsgrad/models/llama.ts:137; the reference flattens and is batch-1 only at this step — the
 * per-row argmax for B>1 is the batched extension the configs ask for).  hidden_out (optional, [B][S][dim]) gets
 * the residual stream after the last block. */
ORC_API int orc_model_forward(orc_model* m, const int32_t* tokens, int B, int S, int start_pos, float* logits_out,
                              int32_t* next_tok, uint16_t* hidden_out) {
  const orc_config* c = &m->c;
  const int d = c->dim, H = c->n_heads, G = c->n_kv_heads, hd = d / H, kv = G * hd, f = c->hidden, V = c->vocab;
  const int R = B * S, T = start_pos + S;
  if (B > c->max_batch || T > c->max_context) return -1;
  h16* h = (h16*)malloc(sizeof(h16) * (size_t)R * d);
  h16* xn = (h16*)malloc(sizeof(h16) * (size_t)R * d);
  h16* q = (h16*)malloc(sizeof(h16) * (size_t)R * d);
  h16* kx = (h16*)malloc(sizeof(h16) * (size_t)R * kv);
  h16* vx = (h16*)malloc(sizeof(h16) * (size_t)R * kv);
  h16* att = (h16*)malloc(sizeof(h16) * (size_t)R * d);
  h16* tmp = (h16*)malloc(sizeof(h16) * (size_t)R * d);
  h16* g1 = (h16*)malloc(sizeof(h16) * (size_t)R * f);
  h16* g3 = (h16*)malloc(sizeof(h16) * (size_t)R * f);
  int32_t* pos = (int32_t*)malloc(sizeof(int32_t) * (size_t)R);
  for (int b = 0; b < B; b++) for (int s = 0; s < S; s++) pos[b * S + s] = start_pos + s;

  if (c->quant_embed) orc_embed_w8(tokens, (const int8_t*)m->glob_w[ORC_TOK_EMB], (const uint16_t*)m->glob_s[ORC_TOK_EMB], (uint16_t*)h, R, d);
  else orc_embed_f16(tokens, (const uint16_t*)m->glob_w[ORC_TOK_EMB], (uint16_t*)h, R, d);

  const size_t cache_b = (size_t)c->max_context * kv;            /* one batch row of K or V */
  const size_t cache_l = (size_t)2 * c->max_batch * cache_b;      /* one layer */
  for (int l = 0; l < c->n_layers; l++) {
    orc_rmsnorm((const uint16_t*)h, (const uint16_t*)m->layer_w[(size_t)l * ORC_PER_LAYER + ORC_ATTN_NORM], (uint16_t*)xn, R, d, c->eps);
    linear_any(m, l, ORC_WQ, xn, q, R, d, d);
    linear_any(m, l, ORC_WK, xn, kx, R, kv, d);
    linear_any(m, l, ORC_WV, xn, vx, R, kv, d);
    orc_rope((uint16_t*)q, (const uint16_t*)m->table, pos, R, H, hd);
    orc_rope((uint16_t*)kx, (const uint16_t*)m->table, pos, R, G, hd);
    h16* kc = m->cache + (size_t)l * cache_l;
    h16* vc = kc + (size_t)c->max_batch * cache_b;
    for (int b = 0; b < B; b++)
      for (int s = 0; s < S; s++) {
        memcpy(kc + (size_t)b * cache_b + (size_t)(start_pos + s) * kv, kx + ((size_t)b * S + s) * kv, (size_t)kv * 2);
        memcpy(vc + (size_t)b * cache_b + (size_t)(start_pos + s) * kv, vx + ((size_t)b * S + s) * kv, (size_t)kv * 2);
      }
    orc_attention((const uint16_t*)q, (const uint16_t*)kc, (const uint16_t*)vc, (uint16_t*)att, B, S, H, G, hd, c->max_context, start_pos);
    linear_any(m, l, ORC_WO, att, tmp, R, d, d);
    for (size_t i = 0; i < (size_t)R * d; i++) h[i] = hadd(h[i], tmp[i]);
    orc_rmsnorm((const uint16_t*)h, (const uint16_t*)m->layer_w[(size_t)l * ORC_PER_LAYER + ORC_FFN_NORM], (uint16_t*)xn, R, d, c->eps);
    linear_any(m, l, ORC_W1, xn, g1, R, f, d);
    linear_any(m, l, ORC_W3, xn, g3, R, f, d);
    for (size_t i = 0; i < (size_t)R * f; i++) g1[i] = silu_mul(g1[i], g3[i]);
    linear_any(m, l, ORC_W2, g1, tmp, R, d, f);
    for (size_t i = 0; i < (size_t)R * d; i++) h[i] = hadd(h[i], tmp[i]);
  }
  if (hidden_out) memcpy(hidden_out, h, sizeof(h16) * (size_t)R * d);

  /* final norm + output on the last position of each batch row (the reference computes all S rows and keeps the
   * last, jsgrad/models/llama.ts:210 — rows are independent, so the kept row is identical) */
  h16* last = (h16*)malloc(sizeof(h16) * (size_t)B * d);
  h16* lastn = (h16*)malloc(sizeof(h16) * (size_t)B * d);
  h16* lg = (h16*)malloc(sizeof(h16) * (size_t)B * V);
  for (int b = 0; b < B; b++) memcpy(last + (size_t)b * d, h + ((size_t)b * S + (S - 1)) * d, (size_t)d * 2);
  orc_rmsnorm((const uint16_t*)last, (const uint16_t*)m->glob_w[ORC_NORM], (uint16_t*)lastn, B, d, c->eps);
  if (c->quant_embed) orc_linear_w8((const uint16_t*)lastn, (const int8_t*)m->glob_w[ORC_OUTPUT], (const uint16_t*)m->glob_s[ORC_OUTPUT], (uint16_t*)lg, B, V, d);
  else orc_linear_f16((const uint16_t*)lastn, (const uint16_t*)m->glob_w[ORC_OUTPUT], (uint16_t*)lg, B, V, d);
  for (int b = 0; b < B; b++) {
    if (logits_out) for (int i = 0; i < V; i++) logits_out[(size_t)b * V + i] = (float)lg[(size_t)b * V + i];
    if (next_tok) next_tok[b] = orc_argmax_f16((const uint16_t*)(lg + (size_t)b * V), V);
  }
  free(h); free(xn); free(q); free(kx); free(vx); free(att); free(tmp); free(g1); free(g3); free(pos);
  free(last); free(lastn); free(lg);
  return 0;
}
