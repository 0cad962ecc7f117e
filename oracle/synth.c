/*
 * synth.c — CPU side of the seeded synthetic-tensor generator used by the parity tests and the CPU baseline.
 *
 * TEST INFRASTRUCTURE ONLY (same rule as llama_oracle.c).  It has no counterpart in the reference: the reference
 * draws random weights with its threefry `Tensor.rand` (jsgrad/tensor.ts:796-843); the workloads here only fix
 * the *distribution* (fp16 ~N(0, 0.02); int8 uniform in [-127,127]; fp16 per-row scales), so a counter-based
 * generator that the device can reproduce bit for bit is used instead:
 *
 *   word(seed, c)  = splitmix64 finaliser of (seed + (c+1) * 0x9E3779B97F4A7C15)
 *   normal element i: S = sum of the twelve 16-bit fields of word(seed,3i), word(seed,3i+1), word(seed,3i+2)
 *                     (Irwin-Hall: mean 12*32767.5, standard deviation 65536 to within 1e-9);
 *                     value = fp16( float(S - 393210) * (std/65536) )     -- one fp32 multiply, one rounding
 *   int8 element i  : (word(seed,i) >> 32) * 255 >> 32, minus 127          -- uniform on [-127,127]
 *   scale element i : fp16( (0.5 + float(word(seed,i) >> 40) * 2^-24) * base )   -- uniform on [0.5,1.5)*base
 *   token i         : (word(seed,i) >> 32) * vocab >> 32
 *
 * Every step is integer arithmetic or a single correctly-rounded fp32 operation, so the CUDA twin in the
 * library yields identical bits.
 */
#include <stdint.h>
#include <string.h>

typedef _Float16 h16;
#define ORC_API __attribute__((visibility("default")))

static inline uint64_t word(uint64_t seed, uint64_t c) {
  uint64_t z = seed + (c + 1) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static inline uint32_t sum16(uint64_t w) {
  return (uint32_t)(w & 0xFFFF) + (uint32_t)((w >> 16) & 0xFFFF) + (uint32_t)((w >> 32) & 0xFFFF) + (uint32_t)(w >> 48);
}

ORC_API void orc_synth_normal_f16(uint64_t seed, uint64_t first, uint64_t n, float std, uint16_t* out) {
  const float c = std / 65536.0f;
#pragma omp parallel for schedule(static)
  for (uint64_t j = 0; j < n; j++) {
    uint64_t i = first + j;
    int32_t S = (int32_t)(sum16(word(seed, 3 * i)) + sum16(word(seed, 3 * i + 1)) + sum16(word(seed, 3 * i + 2)));
    h16 v = (h16)((float)(S - 393210) * c);
    memcpy(out + j, &v, 2);
  }
}
ORC_API void orc_synth_uniform_i8(uint64_t seed, uint64_t first, uint64_t n, int8_t* out) {
#pragma omp parallel for schedule(static)
  for (uint64_t j = 0; j < n; j++) out[j] = (int8_t)((int32_t)(((word(seed, first + j) >> 32) * 255ull) >> 32) - 127);
}
ORC_API void orc_synth_scale_f16(uint64_t seed, uint64_t first, uint64_t n, float base, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (uint64_t j = 0; j < n; j++) {
    float u = 0.5f + (float)(word(seed, first + j) >> 40) * 5.9604644775390625e-08f;
    h16 v = (h16)(u * base);
    memcpy(out + j, &v, 2);
  }
}
ORC_API void orc_synth_const_f16(uint64_t n, float value, uint16_t* out) {
  h16 v = (h16)value;
  for (uint64_t j = 0; j < n; j++) memcpy(out + j, &v, 2);
}
ORC_API void orc_synth_tokens(uint64_t seed, uint64_t first, uint64_t n, int32_t vocab, int32_t* out) {
  for (uint64_t j = 0; j < n; j++) out[j] = (int32_t)(((word(seed, first + j) >> 32) * (uint64_t)vocab) >> 32);
}
