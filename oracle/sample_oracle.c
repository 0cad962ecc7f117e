/*
 * sample_oracle.c — CPU restatement of jsgrad's stochastic `sample` and of the threefry random stream behind
 * `Tensor.rand`.
 *
 * TEST INFRASTRUCTURE ONLY (same rules as llama_oracle.c): the checker the CUDA sampler is compared against; never
 * linked into, imported by or called from the shipped library.  PARITY UNPINNED: the reference holds no expected
 * values for this path and cannot run here; every step below is restated from its source, op by op, in float32 with
 * one rounding per op and no FMA contraction (build with -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

float orc_xexp2_f32(float d); /* llama_oracle.c: the in-tree exp2 polynomial, jsgrad/ops.ts:1650-1673 */

/* Sum of n float32 values in the order the reference's kernels add them: sequentially in ascending index order
 * (jsgrad/codegen/lowerer.ts:130-146); a reduction of 32768 elements or more is first split into `d` contiguous
 * chunks, d the largest divisor of n in [8, 256], each chunk summed sequentially and the d partial sums added in
 * order (UOp.r, jsgrad/ops.ts:433-455). */
ORC_API float orc_sum_f32(const float* x, int n) {
  int d = 0;
  if (n >= 32768)
    for (int c = 256; c >= 8; c--)
      if (n % c == 0) { d = c; break; }
  if (d == 0) {
    float s = 0.0f;
    for (int i = 0; i < n; i++) s = s + x[i];
    return s;
  }
  const int len = n / d;
  float total = 0.0f;
  for (int c = 0; c < d; c++) {
    float s = 0.0f;
    for (int j = 0; j < len; j++) s = s + x[(size_t)c * len + j];
    total = total + s;
  }
  return total;
}

/* Tensor.cumsum along a vector — jsgrad/tensor.ts:2622-2655: every prefix is its own ascending sum; beyond 512
 * elements the vector is padded in front to a multiple of 256, prefix sums are formed inside each block of 256 and
 * the exclusive prefix sums of the block totals are added on top. */
static void cumsum_f32(const float* x, int n, float* out) {
  if (n <= 512) {
    float s = 0.0f;
    for (int i = 0; i < n; i++) { s = s + x[i]; out[i] = s; }
    return;
  }
  const int np = (n + 255) / 256 * 256, pad = np - n, nb = np / 256;
  float* ret = (float*)malloc(sizeof(float) * (size_t)np);
  float* base = (float*)malloc(sizeof(float) * (size_t)nb);
  for (int b = 0; b < nb; b++) {
    float s = 0.0f;
    for (int j = 0; j < 256; j++) {
      const int i = b * 256 + j - pad;
      s = s + (i >= 0 ? x[i] : 0.0f);
      ret[b * 256 + j] = s;
    }
  }
  float run = 0.0f;
  for (int b = 0; b < nb; b++) { base[b] = run; run = run + ret[b * 256 + 255]; }
  for (int i = 0; i < n; i++) out[i] = ret[i + pad] + base[(i + pad) / 256];
  free(ret); free(base);
}

/* Tensor.multinomial (one sample, one row) — jsgrad/tensor.ts:1164-1172: cdf = cumsum(w) * (1 / cumsum(w)[-1]),
 * result = number of cdf entries that the uniform sample is not below. */
static int32_t multinomial_f32(const float* w, int n, float u) {
  float* cw = (float*)malloc(sizeof(float) * (size_t)n);
  cumsum_f32(w, n, cw);
  const float r = 1.0f / cw[n - 1];
  int32_t cnt = 0;
  for (int i = 0; i < n; i++) cnt += (u >= cw[i] * r) ? 1 : 0;
  free(cw);
  return cnt;
}

/*
 * sample — jsgrad/models/llama.ts:131-185.  logits: float32 [n] (the model's fp16 logits widened, :210);
 * alpha_counter: int32 [n] or NULL (the module-level counter of :130, created on first use); u: the uniform sample
 * Tensor.rand would deliver to multinomial.  Returns the token id.
 *   temp < 1e-6           -> argmax, lowest index among equals (:137, jsgrad/tensor.ts:2314-2320)
 *   alpha penalties       -> logits - (counter * af + (counter >= 0) * ap)            (:142-147; `>= 0` as written)
 *   NaN -> -inf, softmax of logits * (1/temp) with the polynomial exp2                  (:150-153)
 *   k > 0: k rounds of (max, lowest index of the max, zero it)                          (:160-167)
 *          approximate top-p on the k survivors: keep entry i while the mass from i to the end, plus everything
 *          outside the top k, is at least 1 - p                                         (:171-173)
 *          multinomial over the kept probabilities, token = kept index                  (:176-177)
 *   k = 0: multinomial over the whole distribution                                      (:179)
 *   the counter of the chosen token is incremented when a penalty is active             (:182)
 */
ORC_API int32_t orc_sample(const float* logits, int n, float temp, int k, float p, float af, float ap,
                           int32_t* alpha_counter, float u) {
  if (temp < 1e-6f) {
    float mx = -INFINITY;
    for (int i = 0; i < n; i++) if (logits[i] > mx) mx = logits[i];
    for (int i = 0; i < n; i++) if (logits[i] == mx) return i;
    return 0;
  }
  const int alpha = (af != 0.0f || ap != 0.0f) && alpha_counter != NULL;
  float* t = (float*)malloc(sizeof(float) * (size_t)n);
  const float inv_temp = (float)(1.0 / (double)temp); /* div = mul by the reciprocal, folded for a constant */
  float mx = -INFINITY;
  for (int i = 0; i < n; i++) {
    float x = logits[i];
    if (alpha) {
      const float pen = (float)alpha_counter[i] * af + (alpha_counter[i] >= 0 ? 1.0f : 0.0f) * ap;
      x = x - pen;
    }
    if (x != x) x = -INFINITY;
    x = x * inv_temp;
    t[i] = x;
    if (x > mx) mx = x;
  }
  const float log2e = (float)(1.0 / 0.6931471805599453); /* 1 / Math.log(2), jsgrad/tensor.ts:2872-2875 */
  for (int i = 0; i < n; i++) t[i] = orc_xexp2_f32((t[i] - mx) * log2e);
  const float r = 1.0f / orc_sum_f32(t, n);
  for (int i = 0; i < n; i++) t[i] = t[i] * r;

  int32_t token;
  if (k > 0) {
    float* out = (float*)calloc((size_t)k, sizeof(float));
    int32_t* idx = (int32_t*)calloc((size_t)k, sizeof(int32_t));
    for (int it = 0; it < k; it++) {
      float tm = -INFINITY;
      for (int i = 0; i < n; i++) if (t[i] > tm) tm = t[i];
      int am = 0;
      for (int i = 0; i < n; i++) if (t[i] == tm) { am = i; break; }
      out[it] = tm; idx[it] = am;
      t[am] = 0.0f;
    }
    const float rest = orc_sum_f32(t, n);
    const float thr = (float)(1.0 - (double)p);
    /* flip -> cumsum -> flip -> + rest: tail[i] = out[k-1] + out[k-2] + ... + out[i] (in that order), + rest */
    float run = 0.0f;
    float* keep_w = (float*)malloc(sizeof(float) * (size_t)k);
    int32_t* keep_i = (int32_t*)malloc(sizeof(int32_t) * (size_t)k);
    for (int i = k - 1; i >= 0; i--) {
      run = run + out[i];
      const int keep = (run + rest) >= thr;
      keep_w[i] = keep ? out[i] : 0.0f;
      keep_i[i] = keep ? idx[i] : 0;
    }
    const int32_t pick = multinomial_f32(keep_w, k, u);
    token = (pick >= 0 && pick < k) ? keep_i[pick] : 0; /* an index past the end gathers nothing: 0 */
    free(out); free(idx); free(keep_w); free(keep_i);
  } else {
    token = multinomial_f32(t, n, u);
  }
  if (alpha && token >= 0 && token < n) alpha_counter[token] += 1;
  free(t);
  return token;
}

/* ------------------------------------------------------------------------------------------------------------
 * threefry2x32 as the reference writes it — jsgrad/ops.ts:1874-1890 — and the random stream of Tensor.rand built
 * on it — jsgrad/tensor.ts:777-782, 796-843.
 * ---------------------------------------------------------------------------------------------------------- */
static inline uint32_t rotl32(uint32_t v, int r) { return (v << r) | (v >> (32 - r)); }

static inline uint64_t threefry2x32(uint64_t x, uint64_t key) {
  static const int rot[2][4] = {{13, 15, 26, 6}, {17, 29, 16, 24}};
  const uint32_t key0 = (uint32_t)key, key1 = (uint32_t)(key >> 32);
  const uint32_t ks[3] = {key1, key0 ^ key1 ^ 0x1BD11BDAu, key0};
  uint32_t x0 = (uint32_t)x + ks[2], x1 = (uint32_t)(x >> 32) + ks[0];
  for (int i = 0; i < 5; i++) {
    for (int j = 0; j < 4; j++) {
      x0 = x0 + x1;
      x1 = x0 ^ rotl32(x1, rot[i % 2][j]);
    }
    x0 = x0 + ks[i % 3];
    x1 = x1 + ks[(i + 1) % 3] + (uint32_t)i + 1u;
  }
  return ((uint64_t)x1 << 32) | (uint64_t)x0;
}

/* Exposed for the known-answer test against the published Threefry-2x32-20 vectors. */
ORC_API uint64_t orc_threefry2x32(uint64_t x, uint64_t key) { return threefry2x32(x, key); }

/* The `num` 32-bit words Tensor.rand draws for a float32 tensor of `num` elements when the device's counter stands
 * at `counter` and its seed pair is (seed0, seed1): word i < ceil(num/2) is the low half of
 * threefry(counts0[i] | counts1[i] << 32), word ceil(num/2) + i its high half, counts0[i] = i + counter,
 * counts1[i] = counts0[i] + ceil(num/2); key = seed1 << 32 | seed0.  out: float32 [num] uniform in [0, 1):
 * mantissa bits from the word's top 23 bits, exponent of 1.0, minus 1. */
ORC_API void orc_threefry_rand_f32(uint32_t seed0, uint32_t seed1, uint32_t counter, uint64_t num, float* out) {
  const uint64_t half = (num + 1) / 2;
  const uint64_t key = ((uint64_t)seed1 << 32) | (uint64_t)seed0;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)half; i++) {
    const uint32_t c0 = (uint32_t)i + counter, c1 = c0 + (uint32_t)half;
    const uint64_t r = threefry2x32(((uint64_t)c1 << 32) | (uint64_t)c0, key);
    const uint32_t lo = (uint32_t)r, hi = (uint32_t)(r >> 32);
    uint32_t b = (lo >> 9) | 0x3F800000u;
    float f;
    memcpy(&f, &b, 4);
    out[i] = f - 1.0f;
    if ((uint64_t)i + half < num) {
      b = (hi >> 9) | 0x3F800000u;
      memcpy(&f, &b, 4);
      out[(uint64_t)i + half] = f - 1.0f;
    }
  }
}
