// Paged KV cache, RoPE + cache write, and decode attention (one new token per batch row) with GQA head sharing.
//
// Attention follows Tensor.scaled_dot_product_attention as the reference graph computes it
// (jsgrad/tensor.ts:3920-3934, softmax :2186-2214): fp32 scores = (q.k) * 1/sqrt(hd); e = exp2((s - max) * 1/ln2)
// with the polynomial exp2; p = half(e * (1/sum e)); out = half(sum_t p_t * v_t) with fp32 accumulation.  Because
// p is rounded to fp16 *after* normalisation, the context is processed in two kernels instead of one online-softmax
// pass: (A) scores, per-split max and sum;  (B) probabilities from the global max/sum, p.v partials, and the
// cross-split combine done by whichever CTA of a (row, kv head) finishes last (ticket counter, no spinning).
// Scores and partials live in a scratch area owned by the cache object.
//
// One CTA serves one (context split, kv head, batch row) and all n_rep query heads that share the kv head
// (repeat_kv: jsgrad/models/llama.ts:34-39, head h uses kv head h / n_rep), so K and V are read once per group.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <cooperative_groups.h>

#include "common.cuh"
#include "kvcache.cuh"
#include "transcendental.cuh"

namespace cg = cooperative_groups;


constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;

struct AttnArgs {
  const __half* qkv;  // [B][qkv_stride], q heads first
  const __half* k_layer;
  const __half* v_layer;
  const int32_t* block_table;
  const int32_t* pos;  // [B]: index of the newest token; attends to [0, pos]
  float* scores;
  float* part_ml;
  float* part_o;
  unsigned int* tickets;
  __half* out;  // [B][H*hd]
  int qkv_stride, H, G, page, page_shift, max_pages_per_seq, n_split, max_ctx;
  int n_pages;  // pages in a caller-owned pool whose block table is checked entry by entry; 0 = validated on the host
  float scale;
};

// Context slice of split j: [t0, t1).  The same arithmetic is used by both kernels and the combine.
__device__ __forceinline__ int attn_chunk(int T, int n_split) {
  int c = (T + n_split - 1) / n_split;
  c = (c + 31) & ~31;
  return c < 32 ? 32 : c;
}


// ------------------------------------------------------------------------------------------------ kernel A
template <int HD, int NREP>
__global__ void __launch_bounds__(ATT_THREADS) attn_scores_kernel(const AttnArgs a) {
  constexpr int LPR = HD / 8;    // lanes per K row (16 B each)
  constexpr int RPW = 32 / LPR;  // rows per warp pass
  constexpr int U = 4;           // row passes in flight
  __shared__ float red[ATT_WARPS][NREP];
  __shared__ float s_m[NREP];
  pdl_launch();
  pdl_wait();
  const int j = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane % LPR, rgrp = lane / LPR;
  const int T = min(max(a.pos[b] + 1, 1), a.max_ctx);  // positions outside the cache are clamped, never followed
  const int chunk = attn_chunk(T, a.n_split);
  const int t0 = j * chunk, t1 = min(T, t0 + chunk);
  float* ml = a.part_ml + (((size_t)b * a.H + (size_t)g * NREP) * a.n_split + j) * 2;  // head r at + r*n_split*2
  if (t0 >= t1) {
    if (tid < NREP) { ml[(size_t)tid * a.n_split * 2 + 0] = -INFINITY; ml[(size_t)tid * a.n_split * 2 + 1] = 0.f; }
    return;
  }
  const int32_t* bt_row = a.block_table + (size_t)b * a.max_pages_per_seq;

  float qf[NREP][8];
#pragma unroll
  for (int r = 0; r < NREP; r++)
    unpack8(ld_128(a.qkv + (size_t)b * a.qkv_stride + (size_t)(g * NREP + r) * HD + sub * 8), qf[r]);

  float lmax[NREP];
#pragma unroll
  for (int r = 0; r < NREP; r++) lmax[r] = -INFINITY;
  float* srow = a.scores + ((size_t)b * a.H + (size_t)g * NREP) * a.max_ctx;  // head r at + r*max_ctx

  // the trip count depends on the CTA's slice only, so every lane takes part in the shuffles below
  for (int base = t0; base < t1; base += ATT_WARPS * RPW * U) {
    const int tb = base + warp * RPW + rgrp;
    uint4 kv[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = tb + u * ATT_WARPS * RPW;
      kv[u] = (t < t1) ? ld_kv_128(kv_row_checked(a.k_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD, a.n_pages), sub * 8)
                       : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = tb + u * ATT_WARPS * RPW;
#pragma unroll
      for (int r = 0; r < NREP; r++) {
        float p = dot8_acc(0.f, kv[u], qf[r]);
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
        const float s = __fmul_rn(p, a.scale);
        if (t < t1) {
          lmax[r] = fmaxf(lmax[r], s);
          if (sub == (r % LPR)) srow[(size_t)r * a.max_ctx + t] = s;
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < NREP; r++) {
    float m = warp_max(lmax[r]);
    if (lane == 0) red[warp][r] = m;
  }
  __syncthreads();
  if (tid < NREP) {
    float m = red[0][tid];
    for (int w = 1; w < ATT_WARPS; w++) m = fmaxf(m, red[w][tid]);
    s_m[tid] = m;
  }
  __syncthreads();
  // second pass over this split's scores: sum of exp relative to the split max
  const float log2e = 1.4426950408889634f;
  float lsum[NREP];
#pragma unroll
  for (int r = 0; r < NREP; r++) lsum[r] = 0.f;
  for (int t = t0 + tid; t < t1; t += ATT_THREADS) {
#pragma unroll
    for (int r = 0; r < NREP; r++)
      lsum[r] = __fadd_rn(lsum[r], jg_xexp2_f32(__fmul_rn(__fsub_rn(srow[(size_t)r * a.max_ctx + t], s_m[r]), log2e)));
  }
  __syncthreads();  // red reuse
#pragma unroll
  for (int r = 0; r < NREP; r++) {
    float s = warp_sum(lsum[r]);
    if (lane == 0) red[warp][r] = s;
  }
  __syncthreads();
  if (tid < NREP) {
    float s = 0.f;
    for (int w = 0; w < ATT_WARPS; w++) s += red[w][tid];
    ml[(size_t)tid * a.n_split * 2 + 0] = s_m[tid];
    ml[(size_t)tid * a.n_split * 2 + 1] = s;
  }
}

// ------------------------------------------------------------------------------------------------ kernel B
template <int HD, int NREP>
__global__ void __launch_bounds__(ATT_THREADS) attn_pv_kernel(const AttnArgs a) {
  constexpr int LPR = HD / 8;
  constexpr int RPW = 32 / LPR;
  constexpr int U = 4;
  static_assert(NREP <= LPR, "one lane per query head of the group computes its probability");
  __shared__ float s_M[NREP], s_rL[NREP];
  __shared__ float part[ATT_WARPS][NREP][HD];
  __shared__ int s_last;
  pdl_launch();
  pdl_wait();
  const int j = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane % LPR, rgrp = lane / LPR;
  const int T = min(max(a.pos[b] + 1, 1), a.max_ctx);  // positions outside the cache are clamped, never followed
  const int chunk = attn_chunk(T, a.n_split);
  const int n_active = (T + chunk - 1) / chunk;
  const int t0 = j * chunk, t1 = min(T, t0 + chunk);
  const size_t head0 = (size_t)b * a.H + (size_t)g * NREP;
  const float log2e = 1.4426950408889634f;

  if (t0 < t1) {
    // global max and normaliser of each head from the per-split statistics: warp r handles head r
    if (warp < NREP) {
      const float* ml = a.part_ml + (head0 + warp) * a.n_split * 2;
      float m = -INFINITY;
      for (int s = lane; s < n_active; s += 32) m = fmaxf(m, ml[s * 2]);
      m = warp_max(m);
      float l = 0.f;
      for (int s = lane; s < n_active; s += 32)
        l = __fadd_rn(l, __fmul_rn(ml[s * 2 + 1], jg_xexp2_f32(__fmul_rn(__fsub_rn(ml[s * 2], m), log2e))));
      l = warp_sum(l);
      if (lane == 0) { s_M[warp] = m; s_rL[warp] = __fdiv_rn(1.0f, l); }
    }
    __syncthreads();

    const int32_t* bt_row = a.block_table + (size_t)b * a.max_pages_per_seq;
    const float* srow = a.scores + head0 * a.max_ctx;
    const int my_r = sub < NREP ? sub : 0;
    const float myM = s_M[my_r], myrL = s_rL[my_r];
    float acc[NREP][8];
#pragma unroll
    for (int r = 0; r < NREP; r++)
#pragma unroll
      for (int i = 0; i < 8; i++) acc[r][i] = 0.f;

    for (int base = t0; base < t1; base += ATT_WARPS * RPW * U) {
      const int tb = base + warp * RPW + rgrp;
      uint4 vv[U];
      float pr[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int t = tb + u * ATT_WARPS * RPW;
        const bool ok = t < t1;
        vv[u] = ok ? ld_kv_128(kv_row_checked(a.v_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD, a.n_pages), sub * 8)
                   : make_uint4(0, 0, 0, 0);
        pr[u] = (ok && sub < NREP) ? srow[(size_t)my_r * a.max_ctx + t] : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        // p = half(e * 1/sum): lane `r` of each row group evaluates head r, then the group shares it
        const float e = jg_xexp2_f32(__fmul_rn(__fsub_rn(pr[u], myM), log2e));
        const float p = __half2float(__float2half_rn(__fmul_rn(e, myrL)));
        float vf[8];
        unpack8(vv[u], vf);
#pragma unroll
        for (int r = 0; r < NREP; r++) {
          const float p_r = __shfl_sync(0xffffffffu, p, rgrp * LPR + r);
#pragma unroll
          for (int i = 0; i < 8; i++) acc[r][i] = fmaf(p_r, vf[i], acc[r][i]);
        }
      }
    }
    // fold the row groups of the warp, then the warps of the CTA
#pragma unroll
    for (int r = 0; r < NREP; r++)
#pragma unroll
      for (int i = 0; i < 8; i++) {
#pragma unroll
        for (int o = 16; o >= LPR; o >>= 1) acc[r][i] += __shfl_xor_sync(0xffffffffu, acc[r][i], o);
      }
    if (rgrp == 0) {
#pragma unroll
      for (int r = 0; r < NREP; r++)
#pragma unroll
        for (int i = 0; i < 8; i++) part[warp][r][sub * 8 + i] = acc[r][i];
    }
    __syncthreads();
    for (int idx = tid; idx < NREP * HD; idx += ATT_THREADS) {
      const int r = idx / HD, i = idx % HD;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; w++) s += part[w][r][i];
      a.part_o[((head0 + r) * a.n_split + j) * HD + i] = s;
    }
  }

  // ---- ticket: the CTA that finishes last for this (row, kv head) sums the active splits in ascending order
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int ticket = atomicAdd(a.tickets + (size_t)b * a.G + g, 1u);
    s_last = (ticket == (unsigned int)(a.n_split - 1));
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = tid; idx < NREP * HD; idx += ATT_THREADS) {
    const int r = idx / HD, i = idx % HD;
    float s = 0.f;
    for (int sp = 0; sp < n_active; sp++) s = __fadd_rn(s, __ldcg(a.part_o + ((head0 + r) * a.n_split + sp) * HD + i));
    a.out[(size_t)b * a.H * HD + (size_t)(g * NREP + r) * HD + i] = __float2half_rn(s);
  }
  if (tid == 0) a.tickets[(size_t)b * a.G + g] = 0u;
}

// ------------------------------------------------------------------------------------------------ RoPE + cache write
// apply_rotary_emb / complex_mult (jsgrad/models/llama.ts:17-32) on the interleaved pairs of Q and K, every op in
// fp16; K and V of the new token go to their page (cache assign, jsgrad/models/llama.ts:87).
// One thread handles 8 consecutive halves (4 pairs) of one head.
__global__ void rope_kvwrite_kernel(__half* __restrict__ qkv, const __half* __restrict__ table,
                                    const int32_t* __restrict__ pos, const int32_t* __restrict__ block_table,
                                    __half* __restrict__ k_layer, __half* __restrict__ v_layer, int B, int H, int G,
                                    int hd, int page, int page_shift, int max_pages_per_seq, int table_rows,
                                    const int32_t* __restrict__ seq, int n_seq) {
  pdl_launch();
  pdl_wait();
  const int per_head = hd / 8;
  const int heads = H + 2 * G;
  const long long total = (long long)B * heads * per_head;
  for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < total; it += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(it % per_head);
    const int h = (int)((it / per_head) % heads);
    const int b = (int)(it / ((long long)per_head * heads));
    const int p = pos[b];
    if (p < 0 || p >= max_pages_per_seq * page || p >= table_rows) continue;  // out-of-range position: leave the row untouched
    const int sq = seq ? seq[b] : b;
    if ((unsigned)sq >= (unsigned)n_seq) continue;  // row mapped to a sequence the block table does not have: skipped too
    __half* src = qkv + ((size_t)b * heads + h) * hd + (size_t)c * 8;
    uint4 raw = *reinterpret_cast<uint4*>(src);
    if (h < H + G) {
      uint4 traw = ld_128(table + ((size_t)p * (hd / 2) + (size_t)c * 4) * 2);
      const __half* x = reinterpret_cast<const __half*>(&raw);
      const __half* t = reinterpret_cast<const __half*>(&traw);
      __align__(16) __half o[8];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const __half xa = x[2 * i], xb = x[2 * i + 1], co = t[2 * i], si = t[2 * i + 1];
        o[2 * i] = hsub1(hmul1(xa, co), hmul1(xb, si));
        o[2 * i + 1] = hadd1(hmul1(xa, si), hmul1(xb, co));
      }
      raw = *reinterpret_cast<uint4*>(o);
    }
    if (h < H) {
      *reinterpret_cast<uint4*>(src) = raw;
    } else {
      const int g = (h < H + G) ? (h - H) : (h - H - G);
      __half* layer = (h < H + G) ? k_layer : v_layer;
      const int pg = block_table[(size_t)sq * max_pages_per_seq + (p >> page_shift)];
      const int slot = p & (page - 1);
      *reinterpret_cast<uint4*>(layer + (((size_t)pg * G + g) * page + slot) * hd + (size_t)c * 8) = raw;
    }
  }
}

// ------------------------------------------------------------------------------------------------ fused decode attention
// RoPE + cache write + attention of one new token per row in ONE launch, for contexts whose scores fit in shared
// memory.  A thread-block cluster of CS CTAs serves one (batch row, kv head); CTA `rank` owns positions
// [rank*chunk, (rank+1)*chunk).  The softmax statistics and the p.v partials cross CTAs through distributed shared
// memory with hardware cluster barriers (no global scratch, no spinning):
//   scores -> local max m_j and local sum l_j of exp2((s-m_j)/ln2) -> cluster: M = max m_j, L = sum l_j exp2((m_j-M)/ln2)
//   -> p = half(exp2((s-M)/ln2) * 1/L) -> local p.v (fp32) -> each rank folds a slice of the outputs over the ranks.
// Every probability is formed from the global max and the global sum and rounded to fp16 before it meets v, as the
// reference's softmax does (jsgrad/tensor.ts:2186-2214); only the order in which the sum is accumulated differs.
// Q is rotated in registers (the qkv buffer keeps the unrotated projection); the CTA that owns the newest position
// rotates K, writes K and V to their page, and then reads them back like any other cached row.
struct AttnFusedArgs {
  const __half* qkv;
  const __half* table;  // [table_rows][hd/2][2]
  __half* k_layer;
  __half* v_layer;
  const int32_t* block_table;
  const int32_t* pos;
  const int32_t* seq;  // row -> sequence (block-table row); null = identity.  Several rows may belong to one sequence
  __half* out;
  int table_rows, qkv_stride, H, G, page, page_shift, max_pages_per_seq, max_ctx, chunk_cap, stages;
  int n_seq;  // rows of the block table: a row whose seq[] entry lies outside [0, n_seq) is skipped (output untouched)
  int pre;  // 1: Q is already rotated and K/V are already in the cache (multi-position calls): attend only
  float scale;
};

template <int HD, int NREP>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_fused_kernel(const AttnFusedArgs a) {
  constexpr int LPR = HD / 8;
  constexpr int RPW = 32 / LPR;
  constexpr int U = 8;                          // row passes in flight
  constexpr int ROWS_IT = ATT_WARPS * RPW * U;  // positions per loop iteration of the CTA
  extern __shared__ __align__(16) float sc[];   // [NREP][chunk_cap] raw scores
  __shared__ float red[ATT_WARPS][NREP];
  __shared__ float s_m[NREP], s_l[NREP], s_M[NREP], s_rL[NREP];
  __shared__ float part[ATT_WARPS][NREP][HD];
  __shared__ float o_part[NREP * HD];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), CS = (int)cluster.num_blocks();
  const int g = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane % LPR, rgrp = lane / LPR;
  pdl_launch();
  pdl_wait();

  const int sq = a.seq ? a.seq[b] : b;
  if ((unsigned)sq >= (unsigned)a.n_seq) return;  // the same for every CTA of the cluster (they share b)
  const int T = min(max(a.pos[b] + 1, 1), a.max_ctx);
  const int p = T - 1;  // position of the new token
  const int chunk = min((T + CS - 1) / CS, a.chunk_cap);  // the host sizes chunk_cap so that CS * chunk_cap >= max_ctx
  const int t0 = rank * chunk, t1 = min(T, t0 + chunk);
  const int32_t* bt_row = a.block_table + (size_t)sq * a.max_pages_per_seq;
  const __half* xrow = a.qkv + (size_t)b * a.qkv_stride;
  const uint4 traw = a.pre ? make_uint4(0, 0, 0, 0)
                           : ld_128(a.table + ((size_t)min(p, a.table_rows - 1) * (HD / 2) + (size_t)sub * 4) * 2);

  // ---- the owner of position p rotates K and stores the new K / V rows
  if (!a.pre && t0 <= p && p < t1 && warp == 0 && lane < LPR) {
    const uint4 kraw = ld_128(xrow + (size_t)(a.H + g) * HD + lane * 8);
    const uint4 vraw = ld_128(xrow + (size_t)(a.H + a.G + g) * HD + lane * 8);
    const int pg = bt_row[p >> a.page_shift], slot = p & (a.page - 1);
    const size_t off = (((size_t)pg * a.G + g) * a.page + slot) * HD + (size_t)lane * 8;
    *reinterpret_cast<uint4*>(a.k_layer + off) = rope8(kraw, traw);
    *reinterpret_cast<uint4*>(a.v_layer + off) = vraw;
  }
  // ---- rotated query slices of the NREP heads of this group
  float qf[NREP][8];
#pragma unroll
  for (int r = 0; r < NREP; r++) {
    const uint4 qraw = ld_128(xrow + (size_t)(g * NREP + r) * HD + sub * 8);
    unpack8(a.pre ? qraw : rope8(qraw, traw), qf[r]);
  }
  __syncthreads();  // the new K / V rows are visible to this CTA's loads below

  // ---- scores of this rank's positions -> shared memory.  The V rows of the first iteration are requested right
  //      after its K rows, so that they travel while the softmax statistics are worked out.
  float lmax[NREP];
#pragma unroll
  for (int r = 0; r < NREP; r++) lmax[r] = -INFINITY;
  uint4 v0[U];
  for (int base = t0; base < t1; base += ROWS_IT) {
    const int tb = base + warp * RPW + rgrp;
    uint4 kv[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = tb + u * ATT_WARPS * RPW;
      kv[u] = (t < t1) ? ld_128(kv_row(a.k_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
    }
    if (base == t0) {
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int t = tb + u * ATT_WARPS * RPW;
        v0[u] = (t < t1) ? ld_128(kv_row(a.v_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = tb + u * ATT_WARPS * RPW;
#pragma unroll
      for (int r = 0; r < NREP; r++) {
        float d = dot8_acc(0.f, kv[u], qf[r]);
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float s = __fmul_rn(d, a.scale);
        if (t < t1) {
          lmax[r] = fmaxf(lmax[r], s);
          if (sub == (r % LPR)) sc[(size_t)r * a.chunk_cap + (t - t0)] = s;
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < NREP; r++) {
    const float m = warp_max(lmax[r]);
    if (lane == 0) red[warp][r] = m;
  }
  __syncthreads();
  if (tid < NREP) {
    float m = red[0][tid];
    for (int w = 1; w < ATT_WARPS; w++) m = fmaxf(m, red[w][tid]);
    s_m[tid] = m;
  }
  __syncthreads();
  // ---- sum of exponentials relative to this rank's own max (combined across ranks below)
  const float log2e = 1.4426950408889634f;
  float lsum[NREP];
#pragma unroll
  for (int r = 0; r < NREP; r++) lsum[r] = 0.f;
  for (int t = t0 + tid; t < t1; t += ATT_THREADS) {
#pragma unroll
    for (int r = 0; r < NREP; r++)
      lsum[r] = __fadd_rn(lsum[r], jg_xexp2_f32(__fmul_rn(__fsub_rn(sc[(size_t)r * a.chunk_cap + (t - t0)], s_m[r]), log2e)));
  }
  __syncthreads();  // `red` is reused
#pragma unroll
  for (int r = 0; r < NREP; r++) {
    const float v = warp_sum(lsum[r]);
    if (lane == 0) red[warp][r] = v;
  }
  __syncthreads();
  if (tid < NREP) {
    float v = 0.f;
    for (int w = 0; w < ATT_WARPS; w++) v += red[w][tid];
    s_l[tid] = v;
  }
  cluster.sync();
  // ---- global max M and normaliser L = sum_j l_j * exp2((m_j - M)/ln2) over the ranks, in rank order
  if (tid < NREP) {
    float M = -INFINITY;
    for (int rk = 0; rk < CS; rk++) M = fmaxf(M, *cluster.map_shared_rank(&s_m[tid], rk));
    float L = 0.f;
    for (int rk = 0; rk < CS; rk++) {
      const float mj = *cluster.map_shared_rank(&s_m[tid], rk), lj = *cluster.map_shared_rank(&s_l[tid], rk);
      L = __fadd_rn(L, __fmul_rn(lj, jg_xexp2_f32(__fmul_rn(__fsub_rn(mj, M), log2e))));
    }
    s_M[tid] = M;
    s_rL[tid] = __fdiv_rn(1.0f, L);
  }
  __syncthreads();

  // ---- p.v over this rank's positions; lane r of each row group evaluates p = half(exp2((s-M)/ln2) * 1/L) of head
  //      r (rounded to fp16 before it meets v, as in the reference graph) and the group shares it
  float acc[NREP][8];
#pragma unroll
  for (int r = 0; r < NREP; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) acc[r][i] = 0.f;
  const int my_r = sub < NREP ? sub : 0;
  const float myM = s_M[my_r], myrL = s_rL[my_r];
  for (int base = t0; base < t1; base += ROWS_IT) {
    const int tb = base + warp * RPW + rgrp;
    uint4 vv[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = tb + u * ATT_WARPS * RPW;
      if (base == t0) vv[u] = v0[u];
      else vv[u] = (t < t1) ? ld_128(kv_row(a.v_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int t = tb + u * ATT_WARPS * RPW;
      const float s = (t < t1 && sub < NREP) ? sc[(size_t)my_r * a.chunk_cap + (t - t0)] : -INFINITY;
      const float e = jg_xexp2_f32(__fmul_rn(__fsub_rn(s, myM), log2e));
      const float pr = __half2float(__float2half_rn(__fmul_rn(e, myrL)));
      float vf[8];
      unpack8(vv[u], vf);
#pragma unroll
      for (int r = 0; r < NREP; r++) {
        const float p_r = __shfl_sync(0xffffffffu, pr, rgrp * LPR + r);
#pragma unroll
        for (int i = 0; i < 8; i++) acc[r][i] = fmaf(p_r, vf[i], acc[r][i]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < NREP; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) {
#pragma unroll
      for (int o = 16; o >= LPR; o >>= 1) acc[r][i] += __shfl_xor_sync(0xffffffffu, acc[r][i], o);
    }
  if (rgrp == 0) {
#pragma unroll
    for (int r = 0; r < NREP; r++)
#pragma unroll
      for (int i = 0; i < 8; i++) part[warp][r][sub * 8 + i] = acc[r][i];
  }
  __syncthreads();
  for (int idx = tid; idx < NREP * HD; idx += ATT_THREADS) {
    const int r = idx / HD, i = idx % HD;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) s += part[w][r][i];
    o_part[idx] = s;
  }
  cluster.sync();

  // ---- each rank folds its slice of the NREP*HD outputs over the ranks, in rank order
  const int per_rank = (NREP * HD + CS - 1) / CS;
  for (int k = tid; k < per_rank; k += ATT_THREADS) {
    const int idx = rank * per_rank + k;
    if (idx < NREP * HD) {
      float s = 0.f;
      for (int rk = 0; rk < CS; rk++) s = __fadd_rn(s, *cluster.map_shared_rank(&o_part[idx], rk));
      a.out[(size_t)b * a.H * HD + (size_t)g * NREP * HD + idx] = __float2half_rn(s);
    }
  }
  cluster.sync();  // peers may still be reading this CTA's shared memory
}

#include "attention_mma.cuh"

// ------------------------------------------------------------------------------------------------ host side

JG_API int jg_kvcache_create(jg_dev* dev, const jg_kvcache_desc* desc, jg_kvcache** out) {
  JG_ENTER(dev);
  JG_REQUIRE(desc != nullptr && out != nullptr, "kvcache_create: null argument");
  const jg_kvcache_desc& d = *desc;
  JG_REQUIRE(d.n_layers > 0 && d.n_kv_heads > 0 && d.n_pages > 0 && d.max_batch > 0 && d.max_pages_per_seq > 0 && d.n_heads > 0,
             "kvcache_create: non-positive dimension");
  JG_REQUIRE(d.head_dim == 64 || d.head_dim == 128, "kvcache_create: head_dim %d not supported (64 or 128)", d.head_dim);
  JG_REQUIRE(d.page_size == 16 || d.page_size == 32 || d.page_size == 64, "kvcache_create: page_size %d not in {16,32,64}", d.page_size);
  JG_REQUIRE(d.n_heads % d.n_kv_heads == 0, "kvcache_create: n_heads %d not a multiple of n_kv_heads %d", d.n_heads, d.n_kv_heads);
  const int n_rep = d.n_heads / d.n_kv_heads;
  JG_REQUIRE(n_rep == 1 || n_rep == 2 || n_rep == 3 || n_rep == 4 || n_rep == 8, "kvcache_create: %d query heads per kv head not supported", n_rep);
  JG_REQUIRE((long long)d.max_batch * d.max_pages_per_seq <= 0x7fffffffLL, "kvcache_create: block table too large");
  jg_kvcache* kv = new jg_kvcache();
  memset(kv, 0, sizeof(*kv));
  kv->dev = dev;
  kv->d = d;
  kv->max_ctx = d.max_pages_per_seq * d.page_size;
  int ns = d.n_split;
  if (ns <= 0) {
    ns = (2 * dev->sm_count + d.max_batch * d.n_kv_heads - 1) / (d.max_batch * d.n_kv_heads);
    const int by_len = (kv->max_ctx + 63) / 64;  // no point in splits shorter than 64 positions at full length
    if (ns > by_len) ns = by_len;
  }
  if (ns < 1) ns = 1;
  if (ns > 64) ns = 64;
  kv->n_split = ns;
  kv->layer_elems = (size_t)d.n_pages * d.n_kv_heads * d.page_size * d.head_dim;
  const size_t pool_bytes = kv->layer_elems * d.n_layers * sizeof(__half);
  const size_t bt_bytes = (size_t)d.max_batch * d.max_pages_per_seq * sizeof(int32_t);
  const size_t sc_bytes = (size_t)d.max_batch * d.n_heads * kv->max_ctx * sizeof(float);
  const size_t ml_bytes = (size_t)d.max_batch * d.n_heads * ns * 2 * sizeof(float);
  const size_t po_bytes = (size_t)d.max_batch * d.n_heads * ns * d.head_dim * sizeof(float);
  const size_t tk_bytes = (size_t)d.max_batch * d.n_kv_heads * sizeof(unsigned int);
  cudaError_t e = cudaSuccess;
  if (e == cudaSuccess) e = cudaMalloc(&kv->k_pool, pool_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->v_pool, pool_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->block_table, bt_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->scores, sc_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->part_ml, ml_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->part_o, po_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->tickets, tk_bytes);
  if (e != cudaSuccess) {
    jg_kvcache_destroy(kv);
    return jg_cuda_fail(e, "cudaMalloc(kv cache)", __FILE__, __LINE__);
  }
  kv->bytes = 2 * pool_bytes + bt_bytes + sc_bytes + ml_bytes + po_bytes + tk_bytes;
  // cache starts as zeros (Tensor.zeros, jsgrad/models/llama.ts:79); tickets must start at zero
  JG_CUDA(cudaMemsetAsync(kv->k_pool, 0, pool_bytes, dev->stream));
  JG_CUDA(cudaMemsetAsync(kv->v_pool, 0, pool_bytes, dev->stream));
  JG_CUDA(cudaMemsetAsync(kv->tickets, 0, tk_bytes, dev->stream));
  // identity block table: row b owns pages [b*mpps, (b+1)*mpps) as far as the pool reaches
  int32_t* bt = (int32_t*)malloc(bt_bytes);
  for (int b = 0; b < d.max_batch; b++)
    for (int i = 0; i < d.max_pages_per_seq; i++) {
      long long pg = (long long)b * d.max_pages_per_seq + i;
      bt[(size_t)b * d.max_pages_per_seq + i] = (int32_t)(pg < d.n_pages ? pg : d.n_pages - 1);
    }
  cudaError_t e2 = cudaMemcpyAsync(kv->block_table, bt, bt_bytes, cudaMemcpyHostToDevice, dev->stream);
  if (e2 == cudaSuccess) e2 = cudaStreamSynchronize(dev->stream);
  free(bt);
  if (e2 != cudaSuccess) {
    jg_kvcache_destroy(kv);
    return jg_cuda_fail(e2, "block table upload", __FILE__, __LINE__);
  }
  *out = kv;
  return JG_OK;
}

static void kvcache_destroy_now(void* p) { jg_kvcache_destroy((jg_kvcache*)p); }

JG_API int jg_kvcache_destroy(jg_kvcache* kv) {
  if (!kv) return JG_OK;
  if (g_jg_capturing > 0) { jg_defer(kvcache_destroy_now, kv); return JG_OK; }
  cudaSetDevice(kv->dev->ordinal);
  cudaStreamSynchronize(kv->dev->stream);
  cudaFree(kv->k_pool); cudaFree(kv->v_pool); cudaFree(kv->block_table); cudaFree(kv->scores);
  cudaFree(kv->part_ml); cudaFree(kv->part_o); cudaFree(kv->tickets);
  delete kv;
  return JG_OK;
}

JG_API int jg_kvcache_set_block_table(jg_kvcache* kv, const int32_t* table) {
  JG_REQUIRE(kv != nullptr && table != nullptr, "kvcache_set_block_table: null argument");
  JG_ENTER(kv->dev);
  const size_t n = (size_t)kv->d.max_batch * kv->d.max_pages_per_seq;
  for (size_t i = 0; i < n; i++)
    JG_REQUIRE(table[i] >= 0 && table[i] < kv->d.n_pages, "kvcache_set_block_table: entry %zu = %d outside the pool of %d pages", i, table[i], kv->d.n_pages);
  JG_CUDA(cudaMemcpyAsync(kv->block_table, table, n * sizeof(int32_t), cudaMemcpyHostToDevice, kv->dev->stream));
  JG_CUDA(cudaStreamSynchronize(kv->dev->stream));
  return JG_OK;
}

JG_API int jg_kvcache_bytes(jg_kvcache* kv, uint64_t* out) {
  JG_REQUIRE(kv != nullptr && out != nullptr, "kvcache_bytes: null argument");
  *out = kv->bytes;
  return JG_OK;
}

static int rope_kvwrite_impl(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t qkv, uint64_t table, int32_t table_rows,
                             uint64_t pos, uint64_t seq, int32_t B, int32_t H);

JG_API int jg_rope_kvwrite(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t qkv, uint64_t table,
                           int32_t table_rows, uint64_t pos, int32_t B, int32_t H) {
  return rope_kvwrite_impl(dev, kv, layer, qkv, table, table_rows, pos, 0, B, H);
}

JG_API int jg_rope_kvwrite_rows(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t qkv, uint64_t table,
                                int32_t table_rows, uint64_t pos, uint64_t seq, int32_t R, int32_t H) {
  JG_REQUIRE(jg_aligned(seq, 4), "rope_kvwrite_rows: null or misaligned row->sequence map");
  return rope_kvwrite_impl(dev, kv, layer, qkv, table, table_rows, pos, seq, R, H);
}

static int rope_kvwrite_impl(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t qkv, uint64_t table, int32_t table_rows,
                             uint64_t pos, uint64_t seq, int32_t B, int32_t H) {
  JG_ENTER(dev);
  JG_REQUIRE(kv != nullptr && kv->dev == dev, "rope_kvwrite: cache belongs to another device");
  JG_REQUIRE(layer >= 0 && layer < kv->d.n_layers, "rope_kvwrite: layer %d out of range", layer);
  JG_REQUIRE(B > 0 && (seq != 0 || B <= kv->d.max_batch) && B <= 65535 && H == kv->d.n_heads, "rope_kvwrite: B=%d H=%d do not match the cache (max_batch %d, n_heads %d)", B, H, kv->d.max_batch, kv->d.n_heads);
  JG_REQUIRE(jg_aligned(qkv, 16) && jg_aligned(table, 16) && jg_aligned(pos, 4), "rope_kvwrite: null or misaligned pointer");
  const int G = kv->d.n_kv_heads, hd = kv->d.head_dim;
  const long long total = (long long)B * (H + 2 * G) * (hd / 8);
  int blocks = (int)((total + 127) / 128);
  if (blocks > dev->sm_count * 8) blocks = dev->sm_count * 8;
  return jg_launch(dev, "rope_kvwrite", rope_kvwrite_kernel, dim3(blocks), dim3(128), 0, (__half*)qkv, (const __half*)table,
                   (const int32_t*)pos, (const int32_t*)kv->block_table, kv->k_pool + kv->layer_elems * layer,
                   kv->v_pool + kv->layer_elems * layer, B, H, G, hd, kv->d.page_size, ilog2(kv->d.page_size),
                   kv->d.max_pages_per_seq, table_rows, (const int32_t*)seq, kv->d.max_batch);
}

template <int HD, int NREP>
static int launch_attn(jg_dev* dev, const AttnArgs& a, int B) {
  dim3 grid(a.n_split, a.G, B);
  int rc = jg_launch(dev, "attn_scores", attn_scores_kernel<HD, NREP>, grid, dim3(ATT_THREADS), 0, a);
  if (rc) return rc;
  return jg_launch(dev, "attn_pv", attn_pv_kernel<HD, NREP>, grid, dim3(ATT_THREADS), 0, a);
}

JG_API int jg_attn_decode(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t pos,
                          int32_t B, int32_t H) {
  JG_ENTER(dev);
  JG_REQUIRE(kv != nullptr && kv->dev == dev, "attn_decode: cache belongs to another device");
  JG_REQUIRE(layer >= 0 && layer < kv->d.n_layers, "attn_decode: layer %d out of range", layer);
  JG_REQUIRE(B > 0 && B <= kv->d.max_batch && H == kv->d.n_heads, "attn_decode: B=%d H=%d do not match the cache (max_batch %d, n_heads %d)", B, H, kv->d.max_batch, kv->d.n_heads);
  JG_REQUIRE(jg_aligned(out, 16) && jg_aligned(qkv, 16) && jg_aligned(pos, 4), "attn_decode: null or misaligned pointer");
  const int G = kv->d.n_kv_heads, hd = kv->d.head_dim, n_rep = H / G;
  AttnArgs a = {};
  a.qkv = (const __half*)qkv;
  a.k_layer = kv->k_pool + kv->layer_elems * layer;
  a.v_layer = kv->v_pool + kv->layer_elems * layer;
  a.block_table = kv->block_table;
  a.pos = (const int32_t*)pos;
  a.scores = kv->scores; a.part_ml = kv->part_ml; a.part_o = kv->part_o; a.tickets = kv->tickets;
  a.out = (__half*)out;
  a.qkv_stride = (H + 2 * G) * hd; a.H = H; a.G = G; a.page = kv->d.page_size; a.page_shift = ilog2(kv->d.page_size);
  a.max_pages_per_seq = kv->d.max_pages_per_seq; a.n_split = kv->n_split; a.max_ctx = kv->max_ctx;
  // 1/sqrt(hd) as the reference folds it: reciprocal of the fp32 constant sqrt(hd) (jsgrad/tensor.ts:3923)
  a.scale = (float)(1.0 / (double)(float)sqrt((double)hd));
#define JG_ATT_CASE(HD_, NR_) if (hd == HD_ && n_rep == NR_) return launch_attn<HD_, NR_>(dev, a, B);
  JG_ATT_CASE(64, 1) JG_ATT_CASE(64, 2) JG_ATT_CASE(64, 3) JG_ATT_CASE(64, 4) JG_ATT_CASE(64, 8)
  JG_ATT_CASE(128, 1) JG_ATT_CASE(128, 2) JG_ATT_CASE(128, 3) JG_ATT_CASE(128, 4) JG_ATT_CASE(128, 8)
#undef JG_ATT_CASE
  jg_set_error("attn_decode: head_dim %d with %d query heads per kv head not supported", hd, n_rep);
  return JG_ENOTSUP;
}

template <int HD, int NREP, bool MMA>
static int launch_attn_fused(jg_dev* dev, const AttnFusedArgs& a, int B, int cs, size_t smem) {
  auto kern = MMA ? attn_decode_mma_kernel<HD, NREP> : attn_decode_fused_kernel<HD, NREP>;
  static size_t smem_set[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int slot = dev->ordinal & 7;
  static bool wide_set[8] = {false, false, false, false, false, false, false, false};
  if (smem > smem_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    smem_set[slot] = smem;
  }
  if (cs > 8 && !wide_set[slot]) {  // clusters of 16 are beyond the portable size: opt in once per kernel and device
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    wide_set[slot] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cs, a.G, B);
  cfg.blockDim = dim3(MMA ? AM_THREADS : ATT_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (dev->pdl && dev->pdl_attn) ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return jg_cuda_fail(e, "attn_decode_fused", __FILE__, __LINE__);
  return jg_after_launch(dev, "attn_decode_fused");
}

static int attn_fused_impl(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t table,
                           int32_t table_rows, uint64_t pos, uint64_t seq, int pre, int32_t B, int32_t H);

JG_API int jg_attn_decode_fused(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t table,
                                int32_t table_rows, uint64_t pos, int32_t B, int32_t H) {
  JG_REQUIRE(jg_aligned(table, 16) && table_rows > 0, "attn_decode_fused: null, misaligned or empty RoPE table");
  return attn_fused_impl(dev, kv, layer, out, qkv, table, table_rows, pos, 0, 0, B, H);
}

JG_API int jg_attn_rows(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t pos, uint64_t seq,
                        int32_t R, int32_t H) {
  JG_REQUIRE(jg_aligned(seq, 4), "attn_rows: null or misaligned row->sequence map");
  return attn_fused_impl(dev, kv, layer, out, qkv, 0, 1, pos, seq, 1, R, H);
}

static int attn_fused_impl(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t table,
                           int32_t table_rows, uint64_t pos, uint64_t seq, int pre, int32_t B, int32_t H) {
  JG_ENTER(dev);
  JG_REQUIRE(kv != nullptr && kv->dev == dev, "attn_decode_fused: cache belongs to another device");
  JG_REQUIRE(layer >= 0 && layer < kv->d.n_layers, "attn_decode_fused: layer %d out of range", layer);
  JG_REQUIRE(B > 0 && (seq != 0 || B <= kv->d.max_batch) && B <= 65535 && H == kv->d.n_heads, "attn_decode_fused: B=%d H=%d do not match the cache (max_batch %d, n_heads %d)", B, H, kv->d.max_batch, kv->d.n_heads);
  JG_REQUIRE(jg_aligned(out, 16) && jg_aligned(qkv, 16) && jg_aligned(pos, 4), "attn_decode_fused: null or misaligned pointer");
  const int G = kv->d.n_kv_heads, hd = kv->d.head_dim, n_rep = H / G;
  static int cluster = -1;
  if (cluster < 0) {
    const char* e = getenv("JG_ATTN_CLUSTER");
    cluster = e ? atoi(e) : 0;
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8 && cluster != 16) cluster = 0;
  }
  // The tensor-core variant of the kernel (attention_mma.cuh) serves launches with 16 or more (row, kv head) pairs;
  // below that the CUDA-core kernel in clusters of 8 is the robust choice.  (Few rows over a short context in clusters
  // of 16 light tensor-core CTAs measured 3.23 against 3.28 ms per step on the 8B shapes but 2.04 against 1.87 on
  // the 3B and 0.92 against 0.84 on the 1B ones.)  JG_ATTN_MMA=0 / 1 and JG_ATTN_CLUSTER force the choice.
  static int mma_env = -2;
  if (mma_env == -2) { const char* e = getenv("JG_ATTN_MMA"); mma_env = e ? (atoi(e) != 0) : -1; }
  // Eight query heads per kv head (70B shapes) fill the MMA's eight columns and overwhelm the CUDA-core kernel's
  // registers: one row over 8200 positions takes 49 us against 95 us.
  const int use_mma = mma_env >= 0 ? mma_env : ((long long)B * G >= 16 || n_rep >= 8);
  static int stages = 0;
  if (!stages) { const char* e = getenv("JG_ATTN_STAGES"); stages = e ? atoi(e) : 2; if (stages < 2 || stages > 4) stages = 2; }
  const size_t tile_bytes = use_mma ? (size_t)stages * AM_TK * (hd + 8) * sizeof(__half) : 0;
  // scores per CTA: rows of chunk_cap floats; the tensor-core variant pads the row so that heads fall on distinct banks
  auto cap_of = [&](int c) { const int per = (kv->max_ctx + c - 1) / c; return use_mma ? (((per + AM_TK - 1) & ~(AM_TK - 1)) + 8) : ((per + 3) & ~3); };
  // CTAs per (row, kv head): as many as it takes to put about two CTAs on every SM, at most 8 — one row alone is
  // latency-bound and wants its context spread widely, many rows fill the machine by themselves and every extra
  // CTA only adds a cluster barrier to a short loop.
  int cs = cluster;
  if (cs == 0) {
    cs = 8;
    if (use_mma) {
      // the tensor-core CTAs are light (4 warps) and the scores of a CTA's positions cost it shared memory, i.e. CTAs
      // per SM: splitting the context keeps more warps and more K / V bytes in flight per SM.  Measured on the 8B shapes
      // (8-layer slices, ms per step for 1 / 2 / 4 / 8 CTAs per pair): 32 rows over 4096 positions 2.46 / 2.54 / 2.14 /
      // 2.24, over 1500 positions 1.65 / - / 1.53 / 1.58, over 512 positions 1.33 / 1.28 / 1.33 / 1.39; 8 rows over 4096
      // positions - / 1.64 / 1.38 / 1.29.  Rule: up to 1024 CTAs, at least 256 positions of the cache's capacity each.
      while (cs > 1 && ((long long)B * G * cs > 1024 || kv->max_ctx / cs < 256)) cs >>= 1;
    } else {
      while (cs > 1 && (long long)B * G * cs > 2LL * dev->sm_count) cs >>= 1;
    }
    // ... but never more positions per CTA than its shared memory can hold scores for
    while (cs < 8 && (size_t)n_rep * cap_of(cs) * sizeof(float) + tile_bytes + 48 * 1024 > (size_t)dev->prop.sharedMemPerBlockOptin) cs <<= 1;
  }
  const int chunk_cap = cap_of(cs);
  const size_t smem = (size_t)n_rep * chunk_cap * sizeof(float) + tile_bytes;
  if (smem + 48 * 1024 > (size_t)dev->prop.sharedMemPerBlockOptin) {
    jg_set_error("attn_decode_fused: %d positions per CTA need %zu B of shared memory; use jg_rope_kvwrite + jg_attn_decode", chunk_cap, smem);
    return JG_ENOTSUP;
  }
  AttnFusedArgs a = {};
  a.qkv = (const __half*)qkv; a.table = (const __half*)table; a.table_rows = table_rows;
  a.k_layer = kv->k_pool + kv->layer_elems * layer; a.v_layer = kv->v_pool + kv->layer_elems * layer;
  a.block_table = kv->block_table; a.pos = (const int32_t*)pos; a.out = (__half*)out;
  a.seq = (const int32_t*)seq; a.pre = pre; a.n_seq = kv->d.max_batch;
  a.qkv_stride = (H + 2 * G) * hd; a.H = H; a.G = G; a.page = kv->d.page_size; a.page_shift = ilog2(kv->d.page_size);
  a.max_pages_per_seq = kv->d.max_pages_per_seq; a.max_ctx = kv->max_ctx; a.chunk_cap = chunk_cap; a.stages = stages;
  a.scale = (float)(1.0 / (double)(float)sqrt((double)hd));
#define JG_ATT_CASE(HD_, NR_)                                                                   \
  if (hd == HD_ && n_rep == NR_)                                                                \
    return use_mma ? launch_attn_fused<HD_, NR_, true>(dev, a, B, cs, smem) : launch_attn_fused<HD_, NR_, false>(dev, a, B, cs, smem);
  JG_ATT_CASE(64, 1) JG_ATT_CASE(64, 2) JG_ATT_CASE(64, 3) JG_ATT_CASE(64, 4) JG_ATT_CASE(64, 8)
  JG_ATT_CASE(128, 1) JG_ATT_CASE(128, 2) JG_ATT_CASE(128, 3) JG_ATT_CASE(128, 4) JG_ATT_CASE(128, 8)
#undef JG_ATT_CASE
  jg_set_error("attn_decode_fused: head_dim %d with %d query heads per kv head not supported", hd, n_rep);
  return JG_ENOTSUP;
}

// ------------------------------------------------------------------------------------------------ no-allocation variant
// jg_attn_decode keeps its scores / split statistics / partial outputs in buffers that jg_kvcache_create obtained
// with cudaMalloc.  Some hosts must not let a kernel library allocate: an engine whose own allocator owns every byte
// of the device and assigns buffers before the kernels run (jsgrad's memory planner and LRU allocator work that way —
// an allocation made behind them is invisible to their accounting and fails once they hold the whole device), or a
// serving loop that cannot afford the device-wide synchronisation a cudaMalloc / cudaFree implies.  For those callers
// this variant takes every input and output from the caller and keeps the scratch in a fixed array that is part of
// the library image: each GPU that loads the library holds JG_NOALLOC_SCRATCH_BYTES of it until the process exits.
constexpr size_t JG_NOALLOC_SCRATCH_BYTES = 8u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[JG_NOALLOC_SCRATCH_BYTES];
// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address: the address is looked up
// once per device (with that device current) and cached here.
static unsigned char* g_noalloc_scratch_addr[64] = {};

static inline size_t align_up_256(size_t v) { return (v + 255) & ~(size_t)255; }

JG_API int jg_attn_decode_noalloc(jg_dev* dev, uint64_t out, uint64_t qkv, uint64_t k_layer, uint64_t v_layer,
                                  uint64_t block_table, uint64_t pos, int32_t B, int32_t H, int32_t G, int32_t head_dim,
                                  int32_t page_size, int32_t max_pages_per_seq, int32_t n_split, int32_t n_pages) {
  JG_ENTER(dev);
  JG_REQUIRE(B > 0 && H > 0 && G > 0 && H % G == 0 && max_pages_per_seq > 0, "attn_decode_noalloc: bad shape B=%d H=%d G=%d pages=%d", B, H, G, max_pages_per_seq);
  JG_REQUIRE(n_pages > 0, "attn_decode_noalloc: the pools hold n_pages=%d pages", n_pages);
  JG_REQUIRE(head_dim == 64 || head_dim == 128, "attn_decode_noalloc: head_dim %d not supported (64 or 128)", head_dim);
  JG_REQUIRE(page_size == 16 || page_size == 32 || page_size == 64, "attn_decode_noalloc: page_size %d not in {16,32,64}", page_size);
  JG_REQUIRE(n_split >= 1 && n_split <= 64, "attn_decode_noalloc: n_split %d outside [1,64]", n_split);
  JG_REQUIRE(jg_aligned(out, 16) && jg_aligned(qkv, 16) && jg_aligned(k_layer, 16) && jg_aligned(v_layer, 16) &&
                 jg_aligned(block_table, 4) && jg_aligned(pos, 4), "attn_decode_noalloc: null or misaligned pointer");
  JG_REQUIRE(dev->ordinal >= 0 && dev->ordinal < 64, "attn_decode_noalloc: device ordinal %d out of range", dev->ordinal);
  const long long max_ctx64 = (long long)max_pages_per_seq * page_size;
  JG_REQUIRE(max_ctx64 <= 0x7fffffffLL, "attn_decode_noalloc: %d pages of %d positions per sequence overflow the context length", max_pages_per_seq, page_size);
  const int n_rep = H / G, max_ctx = (int)max_ctx64;
  // carve the fixed array: scores | (max, sum) per split | partial outputs per split | tickets
  const size_t sc_bytes = align_up_256((size_t)B * H * max_ctx * sizeof(float));
  const size_t ml_bytes = align_up_256((size_t)B * H * n_split * 2 * sizeof(float));
  const size_t po_bytes = align_up_256((size_t)B * H * n_split * head_dim * sizeof(float));
  const size_t tk_bytes = align_up_256((size_t)B * G * sizeof(unsigned int));
  const size_t need = sc_bytes + ml_bytes + po_bytes + tk_bytes;
  if (need > JG_NOALLOC_SCRATCH_BYTES) {
    jg_set_error("attn_decode_noalloc: B=%d H=%d context=%d n_split=%d need %zu bytes of scratch, the built-in array holds %zu; "
                 "use jg_attn_decode with a jg_kvcache for larger shapes", B, H, max_ctx, n_split, need, (size_t)JG_NOALLOC_SCRATCH_BYTES);
    return JG_EINVAL;
  }
  // first call on this device: resolve the device address of the array (dev is current: JG_ENTER set it)
  if (g_noalloc_scratch_addr[dev->ordinal] == nullptr) {
    JG_REQUIRE(!dev->capturing, "attn_decode_noalloc: the first call on a device looks up the scratch array's address and "
               "must come before any graph capture");
    void* p = nullptr;
    JG_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    JG_REQUIRE(p != nullptr, "attn_decode_noalloc: the scratch symbol has no address on device %d", dev->ordinal);
    g_noalloc_scratch_addr[dev->ordinal] = (unsigned char*)p;
  }
  unsigned char* base = g_noalloc_scratch_addr[dev->ordinal];
  AttnArgs a = {};
  a.qkv = (const __half*)qkv;
  a.k_layer = (const __half*)k_layer;
  a.v_layer = (const __half*)v_layer;
  a.block_table = (const int32_t*)block_table;
  a.pos = (const int32_t*)pos;
  a.scores = (float*)base;
  a.part_ml = (float*)(base + sc_bytes);
  a.part_o = (float*)(base + sc_bytes + ml_bytes);
  a.tickets = (unsigned int*)(base + sc_bytes + ml_bytes + po_bytes);
  a.out = (__half*)out;
  a.qkv_stride = (H + 2 * G) * head_dim; a.H = H; a.G = G; a.page = page_size; a.page_shift = ilog2(page_size);
  a.max_pages_per_seq = max_pages_per_seq; a.n_split = n_split; a.max_ctx = max_ctx;
  a.n_pages = n_pages;  // the block table is the caller's and unvalidated: entries outside the pool read as zero rows
  a.scale = (float)(1.0 / (double)(float)sqrt((double)head_dim));
  // the array keeps whatever the last call (of any shape) left in it; only the tickets must start at zero
  JG_CUDA(cudaMemsetAsync(a.tickets, 0, tk_bytes, dev->stream));
#define JG_ATT_CASE(HD_, NR_) if (head_dim == HD_ && n_rep == NR_) return launch_attn<HD_, NR_>(dev, a, B);
  JG_ATT_CASE(64, 1) JG_ATT_CASE(64, 2) JG_ATT_CASE(64, 3) JG_ATT_CASE(64, 4) JG_ATT_CASE(64, 8)
  JG_ATT_CASE(128, 1) JG_ATT_CASE(128, 2) JG_ATT_CASE(128, 3) JG_ATT_CASE(128, 4) JG_ATT_CASE(128, 8)
#undef JG_ATT_CASE
  jg_set_error("attn_decode_noalloc: head_dim %d with %d query heads per kv head not supported", head_dim, n_rep);
  return JG_ENOTSUP;
}
