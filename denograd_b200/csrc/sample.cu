// Stochastic `sample` (jsgrad/models/llama.ts:131-185) as one kernel per call: alpha penalties, NaN masking, softmax of
// logits / temperature, k rounds of (max, lowest index of the max, remove it), the approximate top-p cut on those k,
// and the multinomial draw (jsgrad/tensor.ts:1164-1172) from a uniform sample the caller supplies.
//
// The integer result depends on float32 sums (the softmax normaliser, the mass outside the top k, the cumulative
// sums of the draw), and a float32 sum depends on the order of its additions.  The kernel therefore adds in exactly
// the order the reference's kernels do — ascending within a reduction, reductions of 32768 elements and more first
// split into the largest number of equal contiguous chunks between 8 and 256 (UOp.r, jsgrad/ops.ts:433-455), cumulative
// sums beyond 512 elements in blocks of 256 behind a front pad (Tensor._split_cumalu, jsgrad/tensor.ts:2629-2643) — so
// that the chosen token is the reference's bit for bit, not merely "within rounding".  The chunks / blocks are what
// runs in parallel: one thread per chunk.
//
// One thread-block cluster serves one row of logits: each CTA keeps a contiguous slice of the distribution in shared
// memory (float32), reads the other slices through distributed shared memory where a chunk straddles CTAs, and the
// cluster meets at hardware barriers; no global scratch is used.
#include <math.h>

#include <cooperative_groups.h>

#include "common.cuh"
#include "transcendental.cuh"

namespace cg = cooperative_groups;

constexpr int SMP_THREADS = 1024;
constexpr int SMP_MAX_CLUSTER = 8;
constexpr int SMP_MAXK = 512;      // beyond 512 the reference's cumulative sum changes shape; nobody samples from more
constexpr int SMP_MAX_BLOCKS = 2048;  // 256-element blocks of the k = 0 draw: vocabularies up to 524288

struct SampleArgs {
  const __half* logits;  // [B][V] fp16, widened to fp32 as Transformer.forward does (jsgrad/models/llama.ts:210)
  const float* u;        // [B] uniform samples in [0, 1)
  int32_t* counter;      // [B][V] alpha counters, or null
  int32_t* tokens;       // [B]
  int V, k, per;         // per: elements of the distribution held by one CTA
  int div, len;          // reductions over V: `div` chunks of `len` (div = 0: one sequential pass)
  float inv_temp, thr, af, ap;
};

// Walks the distribution, which is spread over the CTAs' shared-memory slices, in ascending index order.
struct SliceCursor {
  float* const* base;
  int per, owner, off;
  __device__ SliceCursor(float* const* b, int per_, int j) : base(b), per(per_), owner(j / per_), off(j % per_) {}
  __device__ __forceinline__ float load() const { return base[owner][off]; }
  __device__ __forceinline__ void store(float v) const { base[owner][off] = v; }
  __device__ __forceinline__ void next() { if (++off == per) { off = 0; owner++; } }
};

__global__ void __launch_bounds__(SMP_THREADS, 1) sample_kernel(const SampleArgs a) {
  extern __shared__ __align__(16) float tbuf[];  // this CTA's slice of y, then e, then t
  __shared__ float s_red[32];
  __shared__ unsigned long long s_red64[32];
  __shared__ float s_cmax[SMP_MAX_CLUSTER];
  __shared__ unsigned long long s_key[2][SMP_MAX_CLUSTER];
  __shared__ float s_bcast[2];
  __shared__ float s_part[256];
  __shared__ float s_out[SMP_MAXK];
  __shared__ int s_idx[SMP_MAXK];
  __shared__ float s_tot[SMP_MAX_BLOCKS], s_base[SMP_MAX_BLOCKS];
  __shared__ int s_count;
  __shared__ float* s_slices[SMP_MAX_CLUSTER];
  cg::cluster_group cluster = cg::this_cluster();
  const int cr = (int)cluster.block_rank(), cs = (int)cluster.num_blocks();
  const int b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = a.V, per = a.per;
  const int j0 = cr * per, j1 = min(V, j0 + per), nloc = max(j1 - j0, 0);
  pdl_launch();
  pdl_wait();
  if (tid < cs) s_slices[tid] = cluster.map_shared_rank(tbuf, tid);
  if (tid == 0) s_count = 0;
  const float log2e = 1.4426950408889634f;  // (float)(1 / Math.log(2))

  // ---- y = (logit - penalty) * (1 / temperature), NaN -> -inf; maximum over the row
  float lmax = -INFINITY;
  for (int i = tid; i < nloc; i += SMP_THREADS) {
    float x = __half2float(a.logits[(size_t)b * V + j0 + i]);
    if (a.counter != nullptr) {
      const int c = a.counter[(size_t)b * V + j0 + i];
      const float pen = __fadd_rn(__fmul_rn((float)c, a.af), __fmul_rn(c >= 0 ? 1.0f : 0.0f, a.ap));
      x = __fsub_rn(x, pen);
    }
    if (x != x) x = -INFINITY;
    x = __fmul_rn(x, a.inv_temp);
    tbuf[i] = x;
    lmax = fmaxf(lmax, x);
  }
  lmax = warp_max(lmax);
  if (lane == 0) s_red[warp] = lmax;
  __syncthreads();
  if (tid == 0) {
    float m = s_red[0];
    for (int w = 1; w < SMP_THREADS / 32; w++) m = fmaxf(m, s_red[w]);
    for (int c = 0; c < cs; c++) *cluster.map_shared_rank(&s_cmax[cr], c) = m;
  }
  cluster.sync();
  float M = s_cmax[0];
  for (int c = 1; c < cs; c++) M = fmaxf(M, s_cmax[c]);

  // ---- e = exp2((y - M) / ln 2) with the polynomial exp2 (Tensor.exp, jsgrad/tensor.ts:2872-2875)
  for (int i = tid; i < nloc; i += SMP_THREADS) tbuf[i] = jg_xexp2_f32(__fmul_rn(__fsub_rn(tbuf[i], M), log2e));
  cluster.sync();

  // Sum over the whole row in the reference's order; computed by CTA 0, handed to every CTA.  All CTAs call it.
  auto row_sum = [&](int slot) -> float {
    if (cr == 0) {
      if (a.div == 0) {
        if (tid == 0) {
          SliceCursor c(s_slices, per, 0);
          float s = 0.f;
          for (int j = 0; j < V; j++) { s = __fadd_rn(s, c.load()); c.next(); }
          s_part[0] = s;
        }
      } else if (tid < a.div) {
        SliceCursor c(s_slices, per, tid * a.len);
        float s = 0.f;
        for (int j = 0; j < a.len; j++) { s = __fadd_rn(s, c.load()); c.next(); }
        s_part[tid] = s;
      }
      __syncthreads();
      if (tid == 0) {
        float total = s_part[0];
        if (a.div != 0) {
          total = 0.f;
          for (int c = 0; c < a.div; c++) total = __fadd_rn(total, s_part[c]);
        }
        for (int c = 0; c < cs; c++) *cluster.map_shared_rank(&s_bcast[slot], c) = total;
      }
    }
    cluster.sync();
    return s_bcast[slot];
  };

  const float rinv = __fdiv_rn(1.0f, row_sum(0));
  for (int i = tid; i < nloc; i += SMP_THREADS) tbuf[i] = __fmul_rn(tbuf[i], rinv);  // t = e * (1 / sum)
  __syncthreads();

  int token = 0;
  if (a.k > 0) {
    // ---- k rounds: the largest probability and, among equals, its lowest index (the reference's
    //      t.eq(max) * arange(n-1 .. 0) trick); the winner is zeroed.  Probabilities are >= +0, so their bit patterns
    //      order like the values: the key (bits << 32 | ~index) finds both with one unsigned maximum.
    for (int it = 0; it < a.k; it++) {
      unsigned long long best = 0ull;
      for (int i = tid; i < nloc; i += SMP_THREADS) {
        const unsigned long long key = ((unsigned long long)__float_as_uint(tbuf[i]) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)(j0 + i));
        best = key > best ? key : best;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
      }
      if (lane == 0) s_red64[warp] = best;
      __syncthreads();
      if (tid == 0) {
        unsigned long long m = s_red64[0];
        for (int w = 1; w < SMP_THREADS / 32; w++) m = s_red64[w] > m ? s_red64[w] : m;
        for (int c = 0; c < cs; c++) *cluster.map_shared_rank(&s_key[it & 1][cr], c) = m;
      }
      cluster.sync();
      unsigned long long win = s_key[it & 1][0];
      for (int c = 1; c < cs; c++) win = s_key[it & 1][c] > win ? s_key[it & 1][c] : win;
      const int idx = (int)(0xFFFFFFFFu - (uint32_t)(win & 0xFFFFFFFFull));
      if (tid == 0) {
        s_out[it] = __uint_as_float((uint32_t)(win >> 32));
        s_idx[it] = idx;
        if (idx >= j0 && idx < j1) tbuf[idx - j0] = 0.f;
      }
      __syncthreads();
    }
    cluster.sync();  // every removal is visible to the CTA that adds up what is left
    const float rest = row_sum(1);
    if (cr == 0 && tid == 0) {
      // approximate top-p: tail[i] = out[k-1] + ... + out[i] (added in that order) + rest; entry i survives while
      // tail[i] >= 1 - p.  Then the draw: cumulative sums of the survivors, scaled by 1 / total, counted against u.
      const int k = a.k;
      float run = 0.f;
      for (int i = k - 1; i >= 0; i--) {
        run = __fadd_rn(run, s_out[i]);
        const bool keep = __fadd_rn(run, rest) >= a.thr;
        if (!keep) { s_out[i] = 0.f; s_idx[i] = 0; }
      }
      float cw = 0.f;
      for (int i = 0; i < k; i++) cw = __fadd_rn(cw, s_out[i]);
      const float r = __fdiv_rn(1.0f, cw);
      const float u = a.u[b];
      int cnt = 0;
      float acc = 0.f;
      for (int i = 0; i < k; i++) {
        acc = __fadd_rn(acc, s_out[i]);
        cnt += (u >= __fmul_rn(acc, r)) ? 1 : 0;
      }
      token = cnt < k ? s_idx[cnt] : 0;  // an index past the end gathers nothing
    }
  } else {
    // ---- draw from the whole distribution: cumulative sums in blocks of 256 behind a front pad, block totals added
    //      on top, everything scaled by 1 / last, entries not above u counted
    const int np = (V + 255) / 256 * 256, pad = np - V, nb = np / 256;
    const bool blocked = V > 512;
    if (cr == 0) {
      if (blocked) {
        for (int blk = tid; blk < nb; blk += SMP_THREADS) {
          const int first = blk * 256 - pad;  // may be negative in block 0: the pad contributes zeros
          SliceCursor c(s_slices, per, max(first, 0));
          float s = 0.f;
          for (int j = 0; j < 256; j++) {
            if (first + j >= 0) { s = __fadd_rn(s, c.load()); c.store(s); c.next(); }
          }
          s_tot[blk] = s;
        }
        __syncthreads();
        if (tid == 0) {
          float run = 0.f;
          for (int blk = 0; blk < nb; blk++) { s_base[blk] = run; run = __fadd_rn(run, s_tot[blk]); }
        }
      } else if (tid == 0) {
        SliceCursor c(s_slices, per, 0);
        float s = 0.f;
        for (int j = 0; j < V; j++) { s = __fadd_rn(s, c.load()); c.store(s); c.next(); }
      }
      __syncthreads();
      if (tid == 0) {
        SliceCursor c(s_slices, per, V - 1);
        const float last = blocked ? __fadd_rn(c.load(), s_base[nb - 1]) : c.load();
        const float r = __fdiv_rn(1.0f, last);
        for (int q = 0; q < cs; q++) *cluster.map_shared_rank(&s_bcast[1], q) = r;
      }
    }
    cluster.sync();
    const float r = s_bcast[1];
    const float u = a.u[b];
    const float* base0 = cluster.map_shared_rank(s_base, 0);
    int cnt = 0;
    for (int i = tid; i < nloc; i += SMP_THREADS) {
      const float cw = blocked ? __fadd_rn(tbuf[i], base0[(j0 + i + pad) >> 8]) : tbuf[i];
      cnt += (u >= __fmul_rn(cw, r)) ? 1 : 0;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0 && cnt != 0) atomicAdd(cluster.map_shared_rank(&s_count, 0), cnt);
    cluster.sync();
    if (cr == 0 && tid == 0) token = s_count;
  }
  if (cr == 0 && tid == 0) {
    a.tokens[b] = token;
    if (a.counter != nullptr && token >= 0 && token < V) a.counter[(size_t)b * V + token] += 1;
  }
  cluster.sync();  // nobody leaves while a peer may still read its shared memory
}

// Tokens for B rows of fp16 logits [B][V] (device): tokens_out int32 [B]; u float32 [B], one uniform sample in [0, 1)
// per row (what Tensor.rand hands to multinomial); alpha_counter int32 [B][V] or 0.  temp must be >= 1e-6 (below
// that `sample` is an argmax: jg_argmax).  The reference applies `sample` to one flattened row (jsgrad/models/llama.ts:
// 132,212); rows here are independent.
JG_API int jg_sample(jg_dev* dev, uint64_t tokens_out, uint64_t logits, uint64_t u, uint64_t alpha_counter, int32_t B,
                     int32_t V, float temp, int32_t k, float p, float af, float ap) {
  JG_ENTER(dev);
  JG_REQUIRE(B > 0 && B <= 65535 && V > 0, "sample: bad shape B=%d V=%d", B, V);
  JG_REQUIRE(p >= 0.f && p <= 1.f, "sample: p must be between 0 and 1");
  JG_REQUIRE(k >= 0 && k <= V, "sample: k must be between 0 and numel");
  JG_REQUIRE(k <= SMP_MAXK, "sample: k=%d above %d is not implemented", k, SMP_MAXK);
  JG_REQUIRE(temp >= 1e-6f, "sample: temperature below 1e-6 selects argmax (jg_argmax)");
  JG_REQUIRE(jg_aligned(tokens_out, 4) && jg_aligned(logits, 2) && jg_aligned(u, 4) && (alpha_counter == 0 || jg_aligned(alpha_counter, 4)),
             "sample: null or misaligned pointer");
  JG_REQUIRE((V + 255) / 256 <= SMP_MAX_BLOCKS, "sample: a vocabulary of %d exceeds %d", V, SMP_MAX_BLOCKS * 256);
  SampleArgs a = {};
  a.logits = (const __half*)logits; a.u = (const float*)u; a.tokens = (int32_t*)tokens_out;
  a.counter = (af != 0.f || ap != 0.f) ? (int32_t*)alpha_counter : nullptr;
  JG_REQUIRE(!(af != 0.f || ap != 0.f) || alpha_counter != 0, "sample: alpha penalties need the counter buffer");
  a.V = V; a.k = k; a.af = af; a.ap = ap;
  a.inv_temp = (float)(1.0 / (double)temp);
  a.thr = (float)(1.0 - (double)p);
  if (V >= 32768)
    for (int c = 256; c >= 8; c--)
      if (V % c == 0) { a.div = c; a.len = V / c; break; }
  // cluster of 8 (fewer for small rows); every CTA's slice must fit next to the static tables
  int cs = SMP_MAX_CLUSTER;
  while (cs > 1 && V / cs < 2048) cs >>= 1;
  a.per = (V + cs - 1) / cs;
  const size_t smem = (size_t)a.per * sizeof(float);
  const size_t limit = (size_t)dev->prop.sharedMemPerBlockOptin - 40 * 1024;
  if (smem > limit) {
    jg_set_error("sample: %d values per CTA need %zu B of shared memory (limit %zu)", a.per, smem, limit);
    return JG_ENOTSUP;
  }
  static size_t smem_set[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int slot = dev->ordinal & 7;
  if (smem > 48 * 1024 - 40 * 1024 && smem > smem_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit));
    smem_set[slot] = limit;
  }
  return jg_launch_cluster(dev, "sample", sample_kernel, dim3((unsigned)cs, (unsigned)B), dim3(SMP_THREADS), smem, cs, a);
}
