// Device versions of the polynomial exp2 / sin that jsgrad substitutes for EXP2 / SIN on back-ends without native
// transcendentals (jsgrad/ops.ts:1625-1673, helpers :1454-1508).  Written with explicit round-to-nearest
// intrinsics so that no multiply-add pair is contracted: each operation rounds once, as in the reference graph.
#pragma once
#include "common.cuh"

__device__ __forceinline__ float jg_pow2i(int q) { return __int_as_float((q + 127) << 23); }

// xexp2, fp32 branch (jsgrad/ops.ts:1650-1673): q = rintk(x) (add +-0.5, truncate), s = x - q,
// 7-term Horner polynomial, ldexp2k as two power-of-two multiplies, then the range patches.
__device__ __forceinline__ float jg_xexp2_f32(float d) {
  float x = (d != INFINITY) ? ((d != d) ? 0.0f : ((d != -INFINITY) ? d : 0.0f)) : 0.0f;
  int q = (int)__fadd_rn(x, x < 0.0f ? -0.5f : 0.5f);
  float s = __fsub_rn(x, (float)q);
  float u = 0.1535920892e-3f;
  u = __fadd_rn(__fmul_rn(u, s), 0.1339262701e-2f);
  u = __fadd_rn(__fmul_rn(u, s), 0.9618384764e-2f);
  u = __fadd_rn(__fmul_rn(u, s), 0.5550347269e-1f);
  u = __fadd_rn(__fmul_rn(u, s), 0.2402264476e+0f);
  u = __fadd_rn(__fmul_rn(u, s), 0.6931471825e+0f);
  u = __fadd_rn(__fmul_rn(u, s), 1.0f);
  int q1 = q / 2;
  u = __fmul_rn(__fmul_rn(u, jg_pow2i(q1)), jg_pow2i(q - q1));
  if (d >= 128.0f) u = INFINITY;
  if (d < -150.0f) u = 0.0f;
  if (d != d) u = NAN;
  return u;
}

// The same function, bit for bit, for arguments with |d| < 125 only (the caller checks; every score within 86 of its
// row's maximum qualifies): the argument is finite, so the sanitising selects and the range patches are no-ops, and with
// q in [-125, 125] both power-of-two factors and their product 2^q are normal numbers, so scaling the polynomial (a
// value in (0.5, 2)) in one multiply or in two gives the same exact result.  Straight-line code: several calls interleave.
__device__ __forceinline__ float jg_xexp2_f32_mid(float d) {
  const int q = (int)__fadd_rn(d, d < 0.0f ? -0.5f : 0.5f);
  const float s = __fsub_rn(d, (float)q);
  float u = 0.1535920892e-3f;
  u = __fadd_rn(__fmul_rn(u, s), 0.1339262701e-2f);
  u = __fadd_rn(__fmul_rn(u, s), 0.9618384764e-2f);
  u = __fadd_rn(__fmul_rn(u, s), 0.5550347269e-1f);
  u = __fadd_rn(__fmul_rn(u, s), 0.2402264476e+0f);
  u = __fadd_rn(__fmul_rn(u, s), 0.6931471825e+0f);
  u = __fadd_rn(__fmul_rn(u, s), 1.0f);
  return __fmul_rn(u, jg_pow2i(q));
}

// xexp2, fp16 branch: the same graph with every op in fp16 (int16 rintk, bounds 23 / -22).
__device__ __forceinline__ __half jg_xexp2_f16(__half d) {
  const float df = __half2float(d);
  __half x = (df != INFINITY) ? ((df != df) ? __float2half_rn(0.f) : ((df != -INFINITY) ? d : __float2half_rn(0.f)))
                              : __float2half_rn(0.f);
  __half xr = hadd1(x, __float2half_rn(__half2float(x) < 0.0f ? -0.5f : 0.5f));
  float xrf = fminf(fmaxf(__half2float(xr), -32768.0f), 32767.0f);
  int q = (int)xrf;  // truncation; int16 range by the clamp above
  __half s = hsub1(x, __int2half_rn(q));
  __half u = __float2half_rn(0.1535920892e-3f);
  u = hadd1(hmul1(u, s), __float2half_rn(0.1339262701e-2f));
  u = hadd1(hmul1(u, s), __float2half_rn(0.9618384764e-2f));
  u = hadd1(hmul1(u, s), __float2half_rn(0.5550347269e-1f));
  u = hadd1(hmul1(u, s), __float2half_rn(0.2402264476e+0f));
  u = hadd1(hmul1(u, s), __float2half_rn(0.6931471825e+0f));
  u = hadd1(hmul1(u, s), __float2half_rn(1.0f));
  int q1 = q / 2;
  int q2 = q - q1;
  __half p1 = __ushort_as_half((unsigned short)(((q1 + 15) * 1024) & 0xFFFF));
  __half p2 = __ushort_as_half((unsigned short)(((q2 + 15) * 1024) & 0xFFFF));
  u = hmul1(hmul1(u, p1), p2);
  if (df >= 23.0f) u = __float2half_rn(INFINITY);
  if (df < -22.0f) u = __float2half_rn(0.0f);
  if (df != df) u = __float2half_rn(NAN);
  return u;
}

// silu(g) * u in fp16, op by op (jsgrad/tensor.ts:2909-2911,3210-3226; the constant chain
// -1/ln2 * ln2 * 1/ln2 folds to one fp16 constant, jsgrad/ops.ts:1363).
__device__ __forceinline__ __half jg_silu_mul(__half g, __half up) {
  const __half c = __float2half_rn(-1.4426950408889634f);
  __half e = jg_xexp2_f16(hmul1(g, c));
  __half sig = hrecip1(hadd1(__float2half_rn(1.0f), e));
  return hmul1(hmul1(g, sig), up);
}

// sin polynomial on the reduced argument (jsgrad/ops.ts:1596-1605).
__device__ __forceinline__ float jg_sin_poly(float d) {
  float d2 = __fmul_rn(d, d);
  float u = 2.6083159809786593541503e-06f;
  u = __fadd_rn(__fmul_rn(u, d2), -0.0001981069071916863322258f);
  u = __fadd_rn(__fmul_rn(u, d2), 0.00833307858556509017944336f);
  u = __fadd_rn(__fmul_rn(u, d2), -0.166666597127914428710938f);
  u = __fadd_rn(__fmul_rn(u, d2), 1.0f);
  return __fmul_rn(d, u);
}

// xsin, fp32 (jsgrad/ops.ts:1625-1644): Cody-Waite reduction below 30, Payne-Hanek from 30 up.
__device__ __forceinline__ float jg_xsin_f32(float d) {
  float x = (d != INFINITY) ? ((d != d) ? 0.0f : ((d != -INFINITY) ? d : 0.0f)) : 0.0f;
  float x_sign = (x != 0.0f) ? ((x < 0.0f) ? -1.0f : 1.0f) : 0.0f;
  float x_abs = __fmul_rn(x, x_sign);
  float result;
  if (x_abs < 30.0f) {
    // cody_waite_reduction, fp32 branch (jsgrad/ops.ts:1564-1594)
    float t = __fmul_rn(x_abs, 0.318309886183790671537767526745028724f);
    int quad = (int)__fadd_rn(t, t < 0.0f ? -0.5f : 0.5f);
    float qf = (float)quad;
    float v = __fadd_rn(__fmul_rn(qf, -3.1414794921875f), x_abs);
    v = __fadd_rn(__fmul_rn(qf, -0.00011315941810607910156f), v);
    v = __fadd_rn(__fmul_rn(qf, -1.9841872589410058936e-09f), v);
    v = __fadd_rn(__fmul_rn(qf, -1.2154201256553420762e-10f), v);
    float r = jg_sin_poly(v);
    result = __fmul_rn(r, (quad & 1) ? -1.0f : 1.0f);
  } else {
    // payne_hanek_reduction (jsgrad/ops.ts:1513-1558) with frexp (jsgrad/ops.ts:1496-1508)
    const uint32_t two_over_pi_f[7] = {0x00000000u, 0x28be60dbu, 0x9391054au, 0x7f09d5f4u,
                                       0x7d4d3770u, 0x36d8a566u, 0x4f10e410u};
    uint32_t bits = __float_as_uint(x_abs);
    uint32_t exponent = (bits >> 23) & 255u;
    float f = __uint_as_float((bits & 0x807FFFFFu) | 0x3F000000u);
    int e = (int)exponent - 127 + 1;
    unsigned long long ia = (unsigned long long)__fmul_rn(f, 4.294967296e9f);
    unsigned long long i = ((unsigned long long)(long long)e) >> 5;
    e = e & 31;
    int offset = 32 - e;
    uint32_t a[4];
#pragma unroll
    for (int n = 0; n < 4; n++) {
      unsigned long long idx = i + (unsigned long long)n;
      a[n] = two_over_pi_f[idx < 6 ? idx : 6];
    }
    // x << e and x >> offset written as multiply / divide by 2^y in 64 bits, truncated to 32 (`_shl_lazy`,
    // `_shr_lazy`); e in [0,31], offset in [1,32].
    unsigned long long pe = 1ull << e, po = 1ull << offset;
    uint32_t hi = (uint32_t)((unsigned long long)a[0] * pe) | (uint32_t)((unsigned long long)a[1] / po);
    uint32_t mi = (uint32_t)((unsigned long long)a[1] * pe) | (uint32_t)((unsigned long long)a[2] / po);
    uint32_t lo = (uint32_t)((unsigned long long)a[2] * pe) | (uint32_t)((unsigned long long)a[3] / po);
    unsigned long long p = ((ia * (unsigned long long)hi) << 32) + (ia * (unsigned long long)mi) +
                           ((ia * (unsigned long long)lo) >> 32);
    int quad = (int)(p >> 62);
    p &= 0x3fffffffffffffffull;
    float rr = __fmul_rn(__ull2float_rn(p), 3.4061215800865545e-19f);
    float r;
    if (f < 0.5f) { r = rr; }  // the frexp mantissa is always >= 0.5: kept as the source has it
    else { r = __fsub_rn(rr, 1.5707963267948966f); quad = quad + 1; }
    float v = jg_sin_poly(__fadd_rn(r, (quad & 1) ? 1.5707963267948966f : 0.0f));
    result = __fmul_rn(v, (quad & 2) ? -1.0f : 1.0f);
  }
  result = __fmul_rn(result, x_sign);
  if (d == INFINITY || d == -INFINITY || d != d) result = NAN;
  return result;
}
