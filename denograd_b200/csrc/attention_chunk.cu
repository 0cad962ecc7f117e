// Attention for a multi-position chunk (prompt processing): Sc consecutive positions of each of B sequences attend
// causally to the paged KV cache, which already holds the chunk's own K and V (jg_rope_kvwrite_rows ran before).
//
// Arithmetic is Tensor.scaled_dot_product_attention with the additive causal mask of Transformer.forward
// (jsgrad/tensor.ts:3920-3934, softmax :2186-2214, mask jsgrad/models/llama.ts:208): fp32 scores (q.k) * 1/sqrt(hd),
// masked above the diagonal; e = exp2((s - max) * 1/ln2) with the polynomial exp2; p = half(e * (1/sum e));
// out = half(sum_t p_t * v_t) accumulated in fp32.  p is rounded to fp16 *after* normalisation, so the row maximum and
// sum must be known before the first p.v product: the context is walked twice (max and sum together, then p.v),
// recomputing the cheap q.k^T on the tensor cores instead of keeping a [rows][context] score matrix.
//
// One CTA = 16 consecutive positions x the n_rep query heads that share one kv head (repeat_kv,
// jsgrad/models/llama.ts:34-39) of one sequence; warp r owns head r as one m16 tile of mma.sync.m16n8k16 (fp16 in,
// fp32 accumulate), so a K / V tile staged in shared memory serves all n_rep heads.  K and V tiles of 64 positions
// are double-buffered with cp.async.
#include <stdlib.h>

#include "common.cuh"
#include "kvcache.cuh"
#include "transcendental.cuh"

constexpr int CH_Q = 16;   // positions per CTA
constexpr int CH_KV = 64;  // cache positions per staged tile

struct ChunkArgs {
  const __half* qkv;  // [R][qkv_stride], row = s * B + b, q heads first, already rotated
  const __half* k_layer;
  const __half* v_layer;
  const int32_t* block_table;
  const int32_t* pos;  // [R]; pos[s * B + b] = pos[b] + s
  const int32_t* seq;  // [R] row -> block-table row, or null (row b of the chunk is sequence b)
  __half* out;         // [R][H * hd]
  int qkv_stride, H, G, B, Sc, page, page_shift, max_pages_per_seq, max_ctx;
  int n_seq;  // rows of the block table: a sequence whose seq[] entry lies outside [0, n_seq) is skipped
  float scale;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16_zfill(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD, int NREP>
__global__ void __launch_bounds__(NREP * 32, NREP <= 4 ? 3 : 1) attn_chunk_kernel(const ChunkArgs a) {
  constexpr int LD = HD + 8;          // padded row: 32-bit fragment loads and ldmatrix rows fall on distinct banks
  constexpr int NT = NREP * 32;
  constexpr int KS = HD / 16;         // k-steps of q.k^T
  constexpr int NS = CH_KV / 8;       // n-tiles of a score tile
  constexpr int ND = HD / 8;          // n-tiles of the output
  extern __shared__ __align__(16) unsigned char ch_smem[];
  __half* Kb = reinterpret_cast<__half*>(ch_smem);           // [2][CH_KV][LD]
  __half* Vb = Kb + 2 * CH_KV * LD;                          // [2][CH_KV][LD]
  const int tid = threadIdx.x, lane = tid & 31, r = tid >> 5;
  const int qr = lane >> 2, qc = (lane & 3) * 2;             // fragment row / first column of this lane
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;       // long rows first
  const int g = blockIdx.y, b = blockIdx.z;
  pdl_launch();
  pdl_wait();

  const int sq = a.seq ? a.seq[b] : b;
  if ((unsigned)sq >= (unsigned)a.n_seq) return;
  const int pos0 = a.pos[b];
  const int written = min(pos0 + a.Sc, a.max_ctx);           // the cache holds positions [0, written) of this sequence
  const int s0 = qt * CH_Q;                                  // first chunk position of this CTA
  const int p_lo = pos0 + s0;                                // its absolute position
  const int T = min(p_lo + CH_Q, written);                   // positions any row of the tile may attend to
  const int n_tiles = (T + CH_KV - 1) / CH_KV;
  const int32_t* bt_row = a.block_table + (size_t)sq * a.max_pages_per_seq;

  // ---- query fragments of head g*NREP + r: rows qr and qr+8 of the tile (clamped to the chunk)
  uint32_t qf[KS][4];
  {
    const int sa = min(s0 + qr, a.Sc - 1), sb = min(s0 + qr + 8, a.Sc - 1);
    const __half* qa = a.qkv + ((size_t)sa * a.B + b) * a.qkv_stride + (size_t)(g * NREP + r) * HD;
    const __half* qb = a.qkv + ((size_t)sb * a.B + b) * a.qkv_stride + (size_t)(g * NREP + r) * HD;
#pragma unroll
    for (int k = 0; k < KS; k++) {
      qf[k][0] = *reinterpret_cast<const uint32_t*>(qa + k * 16 + qc);
      qf[k][1] = *reinterpret_cast<const uint32_t*>(qb + k * 16 + qc);
      qf[k][2] = *reinterpret_cast<const uint32_t*>(qa + k * 16 + 8 + qc);
      qf[k][3] = *reinterpret_cast<const uint32_t*>(qb + k * 16 + 8 + qc);
    }
  }
  const int prow_a = p_lo + qr, prow_b = p_lo + qr + 8;  // absolute positions of this lane's two rows

  auto load_tile = [&](const __half* layer, int j, __half* dst) {
    for (int idx = tid; idx < CH_KV * (HD / 8); idx += NT) {
      const int row = idx / (HD / 8), c = idx % (HD / 8);
      const int t = j * CH_KV + row;
      const bool ok = t < written;
      const __half* src = ok ? kv_row(layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + c * 8 : layer;
      cp_async_16_zfill(dst + row * LD + c * 8, src, ok);
    }
  };
  // scores of this warp's 16 rows against the 64 positions of tile j: s = (q.k) * scale, -inf above the diagonal
  auto score_tile = [&](const __half* Ks, int j, float (&s)[NS][4]) {
#pragma unroll
    for (int n = 0; n < NS; n++) {
      s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      // B fragments of two k-steps in one ldmatrix: four 8x8 blocks of the 8 positions n*8.., lane l names position
      // n*8 + l%8 at dims 8*(l/8)
      const uint32_t kaddr = (uint32_t)__cvta_generic_to_shared(Ks + (n * 8 + (lane & 7)) * LD + ((lane >> 3) << 3));
#pragma unroll
      for (int k = 0; k < KS; k += 2) {
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(kaddr + k * 32));
        mma_16816(s[n], qf[k], b0, b1);
        mma_16816(s[n], qf[k + 1], b2, b3);
      }
      const int t = j * CH_KV + n * 8 + qc;
      s[n][0] = (t <= prow_a) ? __fmul_rn(s[n][0], a.scale) : -INFINITY;
      s[n][1] = (t + 1 <= prow_a) ? __fmul_rn(s[n][1], a.scale) : -INFINITY;
      s[n][2] = (t <= prow_b) ? __fmul_rn(s[n][2], a.scale) : -INFINITY;
      s[n][3] = (t + 1 <= prow_b) ? __fmul_rn(s[n][3], a.scale) : -INFINITY;
    }
  };

  const float log2e = 1.4426950408889634f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  // ---- pass 1 over K: row maxima and row sums of exp2((s - max) / ln 2), the sums carried relative to the running
  //      maximum and rescaled whenever it grows (the decode kernels combine their context slices the same way)
  load_tile(a.k_layer, 0, Kb);
  cp_async_commit();
#pragma unroll 1
  for (int j = 0; j < n_tiles; j++) {
    if (j + 1 < n_tiles) {
      load_tile(a.k_layer, j + 1, Kb + ((j + 1) & 1) * CH_KV * LD);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float s[NS][4];
    score_tile(Kb + (j & 1) * CH_KV * LD, j, s);
    float t_a = -INFINITY, t_b = -INFINITY;
#pragma unroll
    for (int n = 0; n < NS; n++) {
      t_a = fmaxf(t_a, fmaxf(s[n][0], s[n][1]));
      t_b = fmaxf(t_b, fmaxf(s[n][2], s[n][3]));
    }
    // the four lanes of a quad hold one row between them: they must agree on its maximum
    t_a = fmaxf(t_a, __shfl_xor_sync(0xffffffffu, t_a, 1));
    t_a = fmaxf(t_a, __shfl_xor_sync(0xffffffffu, t_a, 2));
    t_b = fmaxf(t_b, __shfl_xor_sync(0xffffffffu, t_b, 1));
    t_b = fmaxf(t_b, __shfl_xor_sync(0xffffffffu, t_b, 2));
    const float n_a = fmaxf(m_a, t_a), n_b = fmaxf(m_b, t_b);
    if (n_a != m_a) { l_a = __fmul_rn(l_a, jg_xexp2_f32(__fmul_rn(__fsub_rn(m_a, n_a), log2e))); m_a = n_a; }
    if (n_b != m_b) { l_b = __fmul_rn(l_b, jg_xexp2_f32(__fmul_rn(__fsub_rn(m_b, n_b), log2e))); m_b = n_b; }
    // exponents in place of the scores; when the whole warp's lie within (-125, 125) — every tile but the one on the
    // diagonal, whose masked scores are -inf, and rows with a score 86 below their maximum — the short exp2 serves
    bool mid = true;
#pragma unroll
    for (int n = 0; n < NS; n++) {
      s[n][0] = __fmul_rn(__fsub_rn(s[n][0], m_a), log2e); s[n][1] = __fmul_rn(__fsub_rn(s[n][1], m_a), log2e);
      s[n][2] = __fmul_rn(__fsub_rn(s[n][2], m_b), log2e); s[n][3] = __fmul_rn(__fsub_rn(s[n][3], m_b), log2e);
      mid = mid && fabsf(s[n][0]) < 125.0f && fabsf(s[n][1]) < 125.0f && fabsf(s[n][2]) < 125.0f && fabsf(s[n][3]) < 125.0f;
    }
    if (__all_sync(0xffffffffu, mid)) {
#pragma unroll
      for (int n = 0; n < NS; n++) {
        l_a = __fadd_rn(l_a, jg_xexp2_f32_mid(s[n][0])); l_a = __fadd_rn(l_a, jg_xexp2_f32_mid(s[n][1]));
        l_b = __fadd_rn(l_b, jg_xexp2_f32_mid(s[n][2])); l_b = __fadd_rn(l_b, jg_xexp2_f32_mid(s[n][3]));
      }
    } else {
#pragma unroll
      for (int n = 0; n < NS; n++) {
        l_a = __fadd_rn(l_a, jg_xexp2_f32(s[n][0])); l_a = __fadd_rn(l_a, jg_xexp2_f32(s[n][1]));
        l_b = __fadd_rn(l_b, jg_xexp2_f32(s[n][2])); l_b = __fadd_rn(l_b, jg_xexp2_f32(s[n][3]));
      }
    }
    __syncthreads();  // the buffer read here is refilled two iterations on
  }
  l_a = __fadd_rn(l_a, __shfl_xor_sync(0xffffffffu, l_a, 1));
  l_a = __fadd_rn(l_a, __shfl_xor_sync(0xffffffffu, l_a, 2));
  l_b = __fadd_rn(l_b, __shfl_xor_sync(0xffffffffu, l_b, 1));
  l_b = __fadd_rn(l_b, __shfl_xor_sync(0xffffffffu, l_b, 2));
  const float rl_a = __fdiv_rn(1.0f, l_a), rl_b = __fdiv_rn(1.0f, l_b);

  // ---- pass 2: p = half(e * 1/sum) and out += p.v
  float o[ND][4];
#pragma unroll
  for (int n = 0; n < ND; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  load_tile(a.k_layer, 0, Kb);
  load_tile(a.v_layer, 0, Vb);
  cp_async_commit();
#pragma unroll 1
  for (int j = 0; j < n_tiles; j++) {
    if (j + 1 < n_tiles) {
      load_tile(a.k_layer, j + 1, Kb + ((j + 1) & 1) * CH_KV * LD);
      load_tile(a.v_layer, j + 1, Vb + ((j + 1) & 1) * CH_KV * LD);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float s[NS][4];
    score_tile(Kb + (j & 1) * CH_KV * LD, j, s);
    uint32_t pf[CH_KV / 16][4];
    bool mid = true;
#pragma unroll
    for (int n = 0; n < NS; n++) {
      s[n][0] = __fmul_rn(__fsub_rn(s[n][0], m_a), log2e); s[n][1] = __fmul_rn(__fsub_rn(s[n][1], m_a), log2e);
      s[n][2] = __fmul_rn(__fsub_rn(s[n][2], m_b), log2e); s[n][3] = __fmul_rn(__fsub_rn(s[n][3], m_b), log2e);
      mid = mid && fabsf(s[n][0]) < 125.0f && fabsf(s[n][1]) < 125.0f && fabsf(s[n][2]) < 125.0f && fabsf(s[n][3]) < 125.0f;
    }
    if (__all_sync(0xffffffffu, mid)) {  // no masked score in the warp's tile: the short exp2, no zero test
#pragma unroll
      for (int n = 0; n < NS; n++) {
        pf[n >> 1][(n & 1) * 2 + 0] = pack_h2(__fmul_rn(jg_xexp2_f32_mid(s[n][0]), rl_a), __fmul_rn(jg_xexp2_f32_mid(s[n][1]), rl_a));
        pf[n >> 1][(n & 1) * 2 + 1] = pack_h2(__fmul_rn(jg_xexp2_f32_mid(s[n][2]), rl_b), __fmul_rn(jg_xexp2_f32_mid(s[n][3]), rl_b));
      }
    } else {
#pragma unroll
      for (int n = 0; n < NS; n++) {
        const float e0 = jg_xexp2_f32(s[n][0]), e1 = jg_xexp2_f32(s[n][1]), e2 = jg_xexp2_f32(s[n][2]), e3 = jg_xexp2_f32(s[n][3]);
        // masked scores are -inf: force an exact zero so that no unrelated cache row can leak through 0 * x
        const float p0 = s[n][0] == -INFINITY ? 0.f : __fmul_rn(e0, rl_a), p1 = s[n][1] == -INFINITY ? 0.f : __fmul_rn(e1, rl_a);
        const float p2 = s[n][2] == -INFINITY ? 0.f : __fmul_rn(e2, rl_b), p3 = s[n][3] == -INFINITY ? 0.f : __fmul_rn(e3, rl_b);
        pf[n >> 1][(n & 1) * 2 + 0] = pack_h2(p0, p1);
        pf[n >> 1][(n & 1) * 2 + 1] = pack_h2(p2, p3);
      }
    }
    const __half* Vs = Vb + (j & 1) * CH_KV * LD;
#pragma unroll
    for (int kk = 0; kk < CH_KV / 16; kk++) {
      // B fragments of V[16 positions][8 d] come transposed out of ldmatrix: lanes 0-15 name the 16 position rows,
      // lanes 16-31 the same rows 8 columns further (the next n-tile)
      const __half* vrow = Vs + (kk * 16 + (lane & 15)) * LD + ((lane >> 4) * 8);
#pragma unroll
      for (int n = 0; n < ND; n += 2) {
        uint32_t b0, b1, b2, b3;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow + n * 8);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(addr));
        mma_16816(o[n], pf[kk], b0, b1);
        mma_16816(o[n + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();
  }
  // ---- store: rows s0+qr and s0+qr+8 of head g*NREP + r
  const int sa = s0 + qr, sb = s0 + qr + 8;
  __half* oa = a.out + ((size_t)sa * a.B + b) * ((size_t)a.H * HD) + (size_t)(g * NREP + r) * HD;
  __half* ob = a.out + ((size_t)sb * a.B + b) * ((size_t)a.H * HD) + (size_t)(g * NREP + r) * HD;
#pragma unroll
  for (int n = 0; n < ND; n++) {
    if (sa < a.Sc) *reinterpret_cast<uint32_t*>(oa + n * 8 + qc) = pack_h2(o[n][0], o[n][1]);
    if (sb < a.Sc) *reinterpret_cast<uint32_t*>(ob + n * 8 + qc) = pack_h2(o[n][2], o[n][3]);
  }
}

template <int HD, int NREP>
static int launch_chunk(jg_dev* dev, const ChunkArgs& a) {
  auto kern = attn_chunk_kernel<HD, NREP>;
  const size_t smem = (size_t)4 * CH_KV * (HD + 8) * sizeof(__half);
  static bool attr_set[8] = {false, false, false, false, false, false, false, false};
  const int slot = dev->ordinal & 7;
  if (!attr_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[slot] = true;
  }
  dim3 grid((a.Sc + CH_Q - 1) / CH_Q, a.G, a.B);
  return jg_launch(dev, "attn_chunk", kern, grid, dim3(NREP * 32), smem, a);
}

JG_API int jg_attn_chunk(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t pos, uint64_t seq,
                         int32_t B, int32_t Sc, int32_t H) {
  JG_ENTER(dev);
  JG_REQUIRE(kv != nullptr && kv->dev == dev, "attn_chunk: cache belongs to another device");
  JG_REQUIRE(layer >= 0 && layer < kv->d.n_layers, "attn_chunk: layer %d out of range", layer);
  JG_REQUIRE(B > 0 && B <= 65535 && (seq != 0 || B <= kv->d.max_batch) && Sc > 0 && Sc <= kv->max_ctx && H == kv->d.n_heads,
             "attn_chunk: B=%d Sc=%d H=%d do not match the cache (max_batch %d, context %d, n_heads %d)", B, Sc, H,
             kv->d.max_batch, kv->max_ctx, kv->d.n_heads);
  JG_REQUIRE(jg_aligned(out, 16) && jg_aligned(qkv, 16) && jg_aligned(pos, 4) && (seq == 0 || jg_aligned(seq, 4)),
             "attn_chunk: null or misaligned pointer");
  const int G = kv->d.n_kv_heads, hd = kv->d.head_dim, n_rep = H / G;
  ChunkArgs a = {};
  a.qkv = (const __half*)qkv;
  a.k_layer = kv->k_pool + kv->layer_elems * layer;
  a.v_layer = kv->v_pool + kv->layer_elems * layer;
  a.block_table = kv->block_table;
  a.pos = (const int32_t*)pos; a.seq = (const int32_t*)seq; a.out = (__half*)out;
  a.qkv_stride = (H + 2 * G) * hd; a.H = H; a.G = G; a.B = B; a.Sc = Sc;
  a.page = kv->d.page_size; a.page_shift = ilog2(kv->d.page_size);
  a.max_pages_per_seq = kv->d.max_pages_per_seq; a.max_ctx = kv->max_ctx; a.n_seq = kv->d.max_batch;
  a.scale = (float)(1.0 / (double)(float)sqrt((double)hd));  // as the reference folds it (jsgrad/tensor.ts:3923)
#define JG_CH_CASE(HD_, NR_) if (hd == HD_ && n_rep == NR_) return launch_chunk<HD_, NR_>(dev, a);
  JG_CH_CASE(64, 1) JG_CH_CASE(64, 2) JG_CH_CASE(64, 3) JG_CH_CASE(64, 4) JG_CH_CASE(64, 8)
  JG_CH_CASE(128, 1) JG_CH_CASE(128, 2) JG_CH_CASE(128, 3) JG_CH_CASE(128, 4) JG_CH_CASE(128, 8)
#undef JG_CH_CASE
  jg_set_error("attn_chunk: head_dim %d with %d query heads per kv head not supported", hd, n_rep);
  return JG_ENOTSUP;
}
