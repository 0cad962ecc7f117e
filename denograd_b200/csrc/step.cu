// The whole decode step of the Llama forward (jsgrad/models/llama.ts:201-220: embedding, every TransformerBlock, final
// norm, output projection, greedy pick) as ONE persistent kernel — what the reference replays as a captured batch of
// kernels (TinyJit -> GraphRunner, jsgrad/engine/jit.ts:71-141, 273-353) for one token per row.
//
// Why: a decode step of an 8B model is 164 dependent launches of 10-45 us.  Each launch boundary drains the memory
// pipe (tail of the old grid, launch, activation staging, first loads of the new grid: 5-6 us during which HBM idles),
// and at one row per step nothing else is there to hide it: the step sits at 70 % of its HBM roofline although the
// largest kernels stream at 90 %.  Here one CTA per SM stays resident for the whole step (cooperative launch) and the
// kernels become phases separated by grid-wide barriers:
//
//   per layer   P1 x = RMSNorm(h) * g;  qkv = Wqkv x                                   | barrier
//               P2 RoPE(q, k), cache write, scores of this CTA's context slice, slice max / sum -> scratch      | barrier
//               P3 global max / sum, p = half(softmax), p.v partial -> scratch; the last CTA of a (row, kv head)
//                  folds the slices in order into attn                                  | barrier
//               P4 h += Wo attn                                                         | barrier
//               P5 x = RMSNorm(h) * g;  ffn = silu(W1 x) * (W3 x)                       | barrier
//               P6 h += W2 ffn                                                          | barrier
//   per step    x = RMSNorm(h) * g;  logits = Wout x, (value, lowest index) max key     | barrier, pick, feed back
//
// The point of the arrangement is that the weight stream never stops at a phase boundary: weights do not depend on
// activations, so before a CTA arrives at a barrier it has already issued the first two passes of the NEXT projection
// into registers (128 KB per SM in flight), and while the two attention phases run (which move 1 MB at short contexts)
// every CTA has its share of Wo and the head of its W1 / W3 rows brought into L2.
//
// A projection phase: the CTA owns a contiguous run of output rows; its 16 warps split K (thread t owns the 16-byte
// chunks t, t + 512, ... of every row), a pass is 8 loads per lane (R rows x NI chunks x NW matrices), two passes are
// in flight (register double buffer), the per-warp partial sums of a pass meet in shared memory at one barrier per
// pass and are finished in warp order (fixed summation order: results do not depend on timing).
// Arithmetic is that of the stand-alone kernels (gemv.cu, attention.cu): exact fp16 products accumulated in fp32,
// every elementwise fp16 operation rounded once, softmax probabilities formed from the global max and sum and rounded
// to fp16 before they meet v (jsgrad/tensor.ts:2186-2214, 2593-2605; jsgrad/nn/index.ts:586-588).
//
// Every wait on another CTA is bounded (wall clock); a wait that runs out sets the device's error word and the CTA
// leaves the kernel, so a lost CTA ends the launch with JG_ETIMEDOUT at the next synchronisation instead of hanging.
#include "common.cuh"
#include "kvcache.cuh"
#include "transcendental.cuh"

constexpr int ST_THREADS = 512;
constexpr int ST_WARPS = ST_THREADS / 32;
constexpr int ST_PART = 16;  // partial sums per warp and pass: NW * R * MT <= 16

struct StepLayer {
  const __half* attn_norm;
  const __half* wqkv;  // [(H + 2G) * hd][dim]
  const __half* wo;    // [dim][H * hd]
  const __half* ffn_norm;
  const __half* w1;    // [hidden][dim]
  const __half* w3;
  const __half* w2;    // [dim][hidden]
};

struct StepArgs {
  const StepLayer* layers;
  const __half* tok_emb;
  const __half* out_norm;
  const __half* out_w;
  const __half* table;  // RoPE table [table_rows][hd/2][2]
  __half* k_pool;
  __half* v_pool;
  const int32_t* block_table;
  int32_t* tokens;
  int32_t* pos;
  int32_t* next_tokens;  // [n_steps][M]
  __half* h;
  __half* qkv;
  __half* attn;
  __half* ffn;
  __half* logits;
  unsigned long long* key;  // [2] (value, lowest index) max keys of the step's rows (scratch of the plan)
  float* att_ml;          // [M * G][NREP][slices][2]
  float* att_o;           // [M * G][slices][NREP * hd]
  unsigned int* tickets;  // [M * G]
  unsigned int* bar;      // [0] arrivals of the barrier in progress, [32] generation
  int* err;
  size_t layer_elems;
  unsigned long long timeout_ns;
  int n_layers, dim, hidden, H, G, vocab, M, table_rows, page, page_shift, max_pages_per_seq, max_ctx;
  int slices, chunk_cap;  // context slices per (row, kv head) and the scores one slice can hold
  int advance, n_steps;
  int l2_gu_rows;  // rows of W1 / W3 (per CTA) asked into L2 during attention
  float eps, scale, recip_dim;
};

struct StepMat {
  const unsigned char* w[2];
  int r0, r1;  // this CTA's rows
  int KC;      // 16-byte chunks per row
};

__device__ __forceinline__ unsigned long long st_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_cg_128(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// Grid-wide barrier (sense by generation).  All CTAs are resident (cooperative launch).  Returns false when the wait
// ran out; the caller leaves the kernel.
__device__ __forceinline__ bool st_grid_sync(const StepArgs& a, unsigned& gen) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    gen++;
    __threadfence();
    unsigned prev;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(a.bar) : "memory");
    if (prev == gridDim.x - 1) {
      asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(a.bar), "r"(0u) : "memory");
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.bar + 32), "r"(gen) : "memory");
    } else {
      unsigned v;
      unsigned long long t0 = 0;
      unsigned polls = 0;
      for (;;) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.bar + 32) : "memory");
        if (v == gen) break;
        if ((++polls & 255u) == 0) {
          const unsigned long long now = st_now();
          if (t0 == 0) t0 = now;
          else if (now - t0 > a.timeout_ns) { ok = 0; break; }
        }
      }
    }
    __threadfence();
    s_ok = ok;
    if (!ok) atomicCAS(a.err, 0, 4);
  }
  __syncthreads();
  return s_ok != 0;
}

// ---- one pass of a projection: 8 x 16 bytes per lane
template <int R, int NI, int NW>
__device__ __forceinline__ void st_issue(const StepMat& m, int p, uint4 (&b)[8], int tid) {
  static_assert(R * NI * NW == 8, "a pass is 8 loads per lane");
#pragma unroll
  for (int w = 0; w < NW; w++)
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int row = m.r0 + p * R + r;
      const bool rv = row < m.r1;
      const unsigned char* base = m.w[w] + (size_t)(rv ? row : 0) * ((size_t)m.KC * 16);
#pragma unroll
      for (int i = 0; i < NI; i++) {
        const int c = tid + ST_THREADS * i;
        b[(w * R + r) * NI + i] = (rv && c < m.KC) ? ld_stream_128(base + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
      }
    }
}

template <int R, int NI, int NW, int MT>
__device__ __forceinline__ void st_consume(const uint4 (&b)[8], const __half* xs, int K, int KC, float* part, int tid) {
  float acc[NW * R][MT];
#pragma unroll
  for (int j = 0; j < NW * R; j++)
#pragma unroll
    for (int m = 0; m < MT; m++) acc[j][m] = 0.f;
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = tid + ST_THREADS * i;
    if (c < KC) {
#pragma unroll
      for (int m = 0; m < MT; m++) {
        float xf[8];
        unpack8(*reinterpret_cast<const uint4*>(xs + (size_t)m * K + (size_t)c * 8), xf);
#pragma unroll
        for (int j = 0; j < NW * R; j++) acc[j][m] = dot8_acc(acc[j][m], b[j * NI + i], xf);
      }
    }
  }
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int j = 0; j < NW * R; j++)
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const float v = warp_sum(acc[j][m]);
      if (lane == 0) part[warp * ST_PART + j * MT + m] = v;
    }
}

// The phase: on entry wv[0] / wv[1] hold passes 0 / 1 (issued before the preceding barrier); `epi(row, m, s_a, s_b)`
// finishes one output; `next(q, buf)` issues pass q of whatever projection comes next into the buffer that just
// became free.  The pass count is rounded up to an even number >= 2 (empty passes load nothing), so that the next
// projection's passes 0 and 1 always land in wv[0] and wv[1].
template <int R, int NI, int NW, int MT, class Epi, class Next>
__device__ __forceinline__ void st_project(const StepMat& m, const __half* xs, int K, int M, float (*part)[ST_WARPS * ST_PART],
                                           uint4 (&wv)[2][8], int tid, Epi epi, Next next) {
  const int rows = m.r1 - m.r0;
  int np = (rows + R - 1) / R;
  np = np < 2 ? 2 : ((np + 1) & ~1);
  for (int p = 0; p < np; p += 2) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
      st_consume<R, NI, NW, MT>(wv[h], xs, K, m.KC, part[h], tid);
      if (p + 2 + h < np) st_issue<R, NI, NW>(m, p + 2 + h, wv[h], tid);
      else next(h, wv[h]);
      __syncthreads();
      if (tid < R * MT) {
        const int r = tid / MT, mm = tid % MT;
        const int row = m.r0 + (p + h) * R + r;
        if (row < m.r1 && mm < M) {
          float s_a = 0.f, s_b = 0.f;
#pragma unroll
          for (int w = 0; w < ST_WARPS; w++) s_a += part[h][w * ST_PART + r * MT + mm];
          if (NW == 2) {
#pragma unroll
            for (int w = 0; w < ST_WARPS; w++) s_b += part[h][w * ST_PART + (R + r) * MT + mm];
          }
          epi(row, mm, s_a, s_b);
        }
      }
    }
  }
}

template <int MT, int HD, int NREP, int NI_D, int NI_H>
__global__ void __launch_bounds__(ST_THREADS, 1) jg_step_kernel(const StepArgs a) {
  static_assert(NREP <= 4 && MT <= 2, "register budget of 128 per thread");
  constexpr int R_D = 8 / NI_D;  // rows per pass, K = dim
  constexpr int R_H = 8 / NI_H;  // rows per pass, K = hidden
  constexpr int R_G = 4 / NI_D;  // gate/up row pairs per pass
  constexpr int LPR = HD / 8;    // lanes per K / V row
  constexpr int RPW = 32 / LPR;  // rows per warp pass
  constexpr int AU = 2;          // attention row passes in flight
  constexpr int ROWS_IT = ST_WARPS * RPW * AU;

  extern __shared__ __align__(16) unsigned char st_smem[];
  __half* xs = reinterpret_cast<__half*>(st_smem);  // [MT][K] activation rows of a projection phase
  // the attention phases reuse the same bytes: raw scores, per-warp p.v partials, the CTA's p.v partial
  float* sc = reinterpret_cast<float*>(st_smem);                     // [NREP][chunk_cap]
  float* pv_part = sc + (size_t)NREP * a.chunk_cap;                   // [ST_WARPS][NREP][HD]
  float* o_part = pv_part + (size_t)ST_WARPS * NREP * HD;             // [NREP][HD]
  __shared__ float part[2][ST_WARPS * ST_PART];
  __shared__ float red[ST_WARPS][4];
  __shared__ float s_rs[MT];
  __shared__ float s_m[4], s_l[4], s_M[4], s_rL[4];
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bid = blockIdx.x, nb = gridDim.x;
  const int dim = a.dim, hidden = a.hidden, M = a.M;
  const int KC_D = dim / 8, KC_H = hidden / 8;
  const int qkv_dim = (a.H + 2 * a.G) * HD;
  const float log2e = 1.4426950408889634f;

  unsigned gen = 0;
  if (tid == 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(a.bar + 32) : "memory");

  auto mat = [&](const __half* w0, const __half* w1, int N, int KC) {
    StepMat m;
    m.w[0] = reinterpret_cast<const unsigned char*>(w0);
    m.w[1] = reinterpret_cast<const unsigned char*>(w1);
    m.r0 = (int)((long long)bid * N / nb);
    m.r1 = (int)((long long)(bid + 1) * N / nb);
    m.KC = KC;
    return m;
  };
  auto no_next = [](int, uint4 (&)[8]) {};

  // x <- RMSNorm(rows) * g into shared memory (rows beyond M are zero); src(m) = the row's address
  auto stage_norm = [&](auto src, const __half* g) {
    uint4 hv[MT][NI_D];
    float ss[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) {
      ss[m] = 0.f;
      const __half* xg = src(m);
#pragma unroll
      for (int i = 0; i < NI_D; i++) {
        const int c = tid + ST_THREADS * i;
        hv[m][i] = (m < M && xg != nullptr && c < KC_D) ? ld_cg_128(xg + (size_t)c * 8) : make_uint4(0, 0, 0, 0);
        float v[8];
        unpack8(hv[m][i], v);
#pragma unroll
        for (int k = 0; k < 8; k++) ss[m] = fmaf(v[k], v[k], ss[m]);
      }
      ss[m] = warp_sum(ss[m]);
      if (lane == 0) red[warp][m] = ss[m];
    }
    __syncthreads();
    if (tid < MT) {
      float t = 0.f;
      for (int i = 0; i < ST_WARPS; i++) t += red[i][tid];
      s_rs[tid] = sqrtf(__fdiv_rn(1.0f, __fadd_rn(__fmul_rn(t, a.recip_dim), a.eps)));
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const float rs = s_rs[m];
#pragma unroll
      for (int i = 0; i < NI_D; i++) {
        const int c = tid + ST_THREADS * i;
        if (c < KC_D) {
          float v[8];
          unpack8(hv[m][i], v);
          const uint4 gv = ld_128(g + (size_t)c * 8);
          const __half* gh = reinterpret_cast<const __half*>(&gv);
          __align__(16) __half o[8];
#pragma unroll
          for (int k = 0; k < 8; k++) o[k] = hmul1(__float2half_rn(__fmul_rn(v[k], rs)), gh[k]);
          reinterpret_cast<uint4*>(xs + (size_t)m * dim)[c] = *reinterpret_cast<uint4*>(o);
        }
      }
    }
    __syncthreads();
  };
  // x <- rows of a [M][K] buffer another phase wrote
  auto stage_copy = [&](const __half* src, int K) {
    const int kc = K / 8;
    for (int m = 0; m < MT; m++)
      for (int c = tid; c < kc; c += ST_THREADS)
        reinterpret_cast<uint4*>(xs + (size_t)m * K)[c] = (m < M) ? ld_cg_128(src + (size_t)m * K + (size_t)c * 8) : make_uint4(0, 0, 0, 0);
    __syncthreads();
  };

  int tok[MT], posv[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) {
    tok[m] = (m < M) ? a.tokens[m] : 0;
    posv[m] = (m < M) ? a.pos[m] : 0;
  }

  uint4 wv[2][8];
  {
    const StepMat m0 = mat(a.layers[0].wqkv, nullptr, qkv_dim, KC_D);
    st_issue<R_D, NI_D, 1>(m0, 0, wv[0], tid);
    st_issue<R_D, NI_D, 1>(m0, 1, wv[1], tid);
  }

  for (int step = 0; step < a.n_steps; step++) {
    for (int l = 0; l < a.n_layers; l++) {
      const StepLayer* L = a.layers + l;
      // ================================================================ P1: norm -> qkv
      if (l == 0) {
        // the embedding rows are the block's input (a token outside the table matches no row: zeros); CTA 0 stores them
        // as the residual stream
        auto emb = [&](int m) -> const __half* {
          return ((unsigned)tok[m] < (unsigned)a.vocab) ? a.tok_emb + (size_t)tok[m] * dim : nullptr;
        };
        if (bid == 0) {
          for (int m = 0; m < M; m++)
            for (int c = tid; c < KC_D; c += ST_THREADS) {
              const __half* e = emb(m);
              reinterpret_cast<uint4*>(a.h + (size_t)m * dim)[c] = e ? ld_128(e + (size_t)c * 8) : make_uint4(0, 0, 0, 0);
            }
        }
        stage_norm(emb, L->attn_norm);
      } else {
        stage_norm([&](int m) -> const __half* { return a.h + (size_t)m * dim; }, L->attn_norm);
      }
      {
        const StepMat mq = mat(L->wqkv, nullptr, qkv_dim, KC_D);
        st_project<R_D, NI_D, 1, MT>(mq, xs, dim, M, part, wv, tid,
                                     [&](int row, int m, float s, float) { a.qkv[(size_t)m * qkv_dim + row] = __float2half_rn(s); },
                                     no_next);
      }
      // while attention runs the memory pipe is idle: this CTA's rows of Wo and the head of its W1 / W3 rows -> L2
      {
        const StepMat mo = mat(L->wo, nullptr, dim, KC_D);
        const uint32_t rb = (uint32_t)KC_D * 16u;
        for (int r = mo.r0 + tid; r < mo.r1; r += ST_THREADS)
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(mo.w[0] + (size_t)r * rb), "r"(rb) : "memory");
        const StepMat mg = mat(L->w1, L->w3, hidden, KC_D);
        const int ng = min(a.l2_gu_rows, mg.r1 - mg.r0);
        for (int r = tid; r < 2 * ng; r += ST_THREADS)
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(mg.w[r & 1] + (size_t)(mg.r0 + (r >> 1)) * rb), "r"(rb) : "memory");
      }
      if (!st_grid_sync(a, gen)) return;
      if (l == 0 && bid == 0 && tid < M) a.key[tid] = 0ull;  // every CTA has read the previous step's key by now

      // ================================================================ P2: RoPE, cache write, scores of a context slice
      const int n_pairs = M * a.G;
      const bool att = bid < n_pairs * a.slices;
      const int pair = att ? bid / a.slices : 0, slice = att ? bid % a.slices : 0;
      const int b = pair / a.G, g = pair % a.G;
      const int sub = lane % LPR, rgrp = lane / LPR;
      int pb = posv[0];
#pragma unroll
      for (int m = 1; m < MT; m++) pb = (b == m) ? posv[m] : pb;
      const int T = min(max(pb + 1, 1), a.max_ctx);
      const int pnew = T - 1;
      const int chunk = min((T + a.slices - 1) / a.slices, a.chunk_cap);
      const int t0 = slice * chunk, t1 = att ? min(T, t0 + chunk) : t0;
      const int32_t* bt_row = a.block_table + (size_t)b * a.max_pages_per_seq;
      __half* k_layer = a.k_pool + (size_t)l * a.layer_elems;
      __half* v_layer = a.v_pool + (size_t)l * a.layer_elems;
      uint4 v0[AU];
      if (att) {
        const __half* xrow = a.qkv + (size_t)b * qkv_dim;
        const uint4 traw = ld_128(a.table + ((size_t)min(pnew, a.table_rows - 1) * (HD / 2) + (size_t)sub * 4) * 2);
        if (t0 <= pnew && pnew < t1 && warp == 0 && lane < LPR) {
          const uint4 kraw = ld_cg_128(xrow + (size_t)(a.H + g) * HD + lane * 8);
          const uint4 vraw = ld_cg_128(xrow + (size_t)(a.H + a.G + g) * HD + lane * 8);
          const int pg = bt_row[pnew >> a.page_shift], slot = pnew & (a.page - 1);
          const size_t off = (((size_t)pg * a.G + g) * a.page + slot) * HD + (size_t)lane * 8;
          *reinterpret_cast<uint4*>(k_layer + off) = rope8(kraw, traw);
          *reinterpret_cast<uint4*>(v_layer + off) = vraw;
        }
        float qf[NREP][8];
#pragma unroll
        for (int r = 0; r < NREP; r++) unpack8(rope8(ld_cg_128(xrow + (size_t)(g * NREP + r) * HD + sub * 8), traw), qf[r]);
        __syncthreads();  // the new K / V rows are visible to this CTA's loads below
        float lmax[NREP];
#pragma unroll
        for (int r = 0; r < NREP; r++) lmax[r] = -INFINITY;
        for (int base = t0; base < t1; base += ROWS_IT) {
          const int tb = base + warp * RPW + rgrp;
          uint4 kk[AU];
#pragma unroll
          for (int u = 0; u < AU; u++) {
            const int t = tb + u * ST_WARPS * RPW;
            kk[u] = (t < t1) ? ld_cg_128(kv_row(k_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
          }
          if (base == t0) {
#pragma unroll
            for (int u = 0; u < AU; u++) {
              const int t = tb + u * ST_WARPS * RPW;
              v0[u] = (t < t1) ? ld_cg_128(kv_row(v_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
            }
          }
#pragma unroll
          for (int u = 0; u < AU; u++) {
            const int t = tb + u * ST_WARPS * RPW;
#pragma unroll
            for (int r = 0; r < NREP; r++) {
              float d = dot8_acc(0.f, kk[u], qf[r]);
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
          const float mx = warp_max(lmax[r]);
          if (lane == 0) red[warp][r] = mx;
        }
        __syncthreads();
        if (tid < NREP) {
          float mx = red[0][tid];
          for (int w = 1; w < ST_WARPS; w++) mx = fmaxf(mx, red[w][tid]);
          s_m[tid] = mx;
        }
        __syncthreads();
        float lsum[NREP];
#pragma unroll
        for (int r = 0; r < NREP; r++) lsum[r] = 0.f;
        for (int t = t0 + tid; t < t1; t += ST_THREADS) {
#pragma unroll
          for (int r = 0; r < NREP; r++)
            lsum[r] = __fadd_rn(lsum[r], jg_xexp2_f32(__fmul_rn(__fsub_rn(sc[(size_t)r * a.chunk_cap + (t - t0)], s_m[r]), log2e)));
        }
#pragma unroll
        for (int r = 0; r < NREP; r++) {
          const float v = warp_sum(lsum[r]);
          if (lane == 0) red[warp][r] = v;
        }
        __syncthreads();
        if (tid < NREP) {
          float v = 0.f;
          for (int w = 0; w < ST_WARPS; w++) v += red[w][tid];
          float* ml = a.att_ml + (((size_t)pair * NREP + tid) * a.slices + slice) * 2;
          ml[0] = s_m[tid];
          ml[1] = v;
        }
      }
      if (!st_grid_sync(a, gen)) return;

      // ================================================================ P3: probabilities, p.v, fold over the slices
      if (att) {
        if (tid < NREP) {
          const float* ml = a.att_ml + ((size_t)pair * NREP + tid) * a.slices * 2;
          float Mx = -INFINITY;
          for (int j = 0; j < a.slices; j++) Mx = fmaxf(Mx, __ldcg(ml + 2 * j));
          float Ls = 0.f;
          for (int j = 0; j < a.slices; j++) {
            const float mj = __ldcg(ml + 2 * j), lj = __ldcg(ml + 2 * j + 1);
            Ls = __fadd_rn(Ls, __fmul_rn(lj, jg_xexp2_f32(__fmul_rn(__fsub_rn(mj, Mx), log2e))));
          }
          s_M[tid] = Mx;
          s_rL[tid] = __fdiv_rn(1.0f, Ls);
        }
        __syncthreads();
        float acc[NREP][8];
#pragma unroll
        for (int r = 0; r < NREP; r++)
#pragma unroll
          for (int i = 0; i < 8; i++) acc[r][i] = 0.f;
        const int my_r = sub < NREP ? sub : 0;
        const float myM = s_M[my_r], myrL = s_rL[my_r];
        for (int base = t0; base < t1; base += ROWS_IT) {
          const int tb = base + warp * RPW + rgrp;
          uint4 vv[AU];
#pragma unroll
          for (int u = 0; u < AU; u++) {
            const int t = tb + u * ST_WARPS * RPW;
            if (base == t0) vv[u] = v0[u];
            else vv[u] = (t < t1) ? ld_cg_128(kv_row(v_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int u = 0; u < AU; u++) {
            const int t = tb + u * ST_WARPS * RPW;
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
            for (int i = 0; i < 8; i++) pv_part[((size_t)warp * NREP + r) * HD + sub * 8 + i] = acc[r][i];
        }
        __syncthreads();
        float* po = a.att_o + ((size_t)pair * a.slices + slice) * (NREP * HD);
        for (int idx = tid; idx < NREP * HD; idx += ST_THREADS) {
          float s = 0.f;
#pragma unroll
          for (int w = 0; w < ST_WARPS; w++) s += pv_part[(size_t)w * NREP * HD + idx];
          po[idx] = s;
        }
        // the last CTA of the pair to get here folds the slices in slice order
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          unsigned prev;
          asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(a.tickets + pair) : "memory");
          s_last = (prev == (unsigned)a.slices - 1u);
          if (s_last) a.tickets[pair] = 0;
          __threadfence();
        }
        __syncthreads();
        if (s_last) {
          const float* pall = a.att_o + (size_t)pair * a.slices * (NREP * HD);
          for (int idx = tid; idx < NREP * HD; idx += ST_THREADS) {
            float s = 0.f;
            for (int j = 0; j < a.slices; j++) s = __fadd_rn(s, __ldcg(pall + (size_t)j * (NREP * HD) + idx));
            a.attn[(size_t)b * a.H * HD + (size_t)g * NREP * HD + idx] = __float2half_rn(s);
          }
        }
      }
      {
        const StepMat mo = mat(L->wo, nullptr, dim, KC_D);
        st_issue<R_D, NI_D, 1>(mo, 0, wv[0], tid);
        st_issue<R_D, NI_D, 1>(mo, 1, wv[1], tid);
      }
      if (!st_grid_sync(a, gen)) return;

      // ================================================================ P4: h += Wo attn
      stage_copy(a.attn, dim);
      {
        const StepMat mo = mat(L->wo, nullptr, dim, KC_D);
        const StepMat mg = mat(L->w1, L->w3, hidden, KC_D);
        st_project<R_D, NI_D, 1, MT>(mo, xs, dim, M, part, wv, tid,
                                     [&](int row, int m, float s, float) {
                                       __half* hp = a.h + (size_t)m * dim + row;
                                       *hp = hadd1(__ldcg(hp), __float2half_rn(s));
                                     },
                                     [&](int q, uint4 (&buf)[8]) { st_issue<R_G, NI_D, 2>(mg, q, buf, tid); });
      }
      if (!st_grid_sync(a, gen)) return;

      // ================================================================ P5: norm -> silu(W1 x) * (W3 x)
      stage_norm([&](int m) -> const __half* { return a.h + (size_t)m * dim; }, L->ffn_norm);
      {
        const StepMat mg = mat(L->w1, L->w3, hidden, KC_D);
        const StepMat md = mat(L->w2, nullptr, dim, KC_H);
        st_project<R_G, NI_D, 2, MT>(mg, xs, dim, M, part, wv, tid,
                                     [&](int row, int m, float sa, float sb) {
                                       a.ffn[(size_t)m * hidden + row] = jg_silu_mul(__float2half_rn(sa), __float2half_rn(sb));
                                     },
                                     [&](int q, uint4 (&buf)[8]) { st_issue<R_H, NI_H, 1>(md, q, buf, tid); });
      }
      if (!st_grid_sync(a, gen)) return;

      // ================================================================ P6: h += W2 ffn
      stage_copy(a.ffn, hidden);
      {
        const StepMat md = mat(L->w2, nullptr, dim, KC_H);
        const bool more = l + 1 < a.n_layers;
        const StepMat mn = more ? mat(a.layers[l + 1].wqkv, nullptr, qkv_dim, KC_D) : mat(a.out_w, nullptr, a.vocab, KC_D);
        st_project<R_H, NI_H, 1, MT>(md, xs, hidden, M, part, wv, tid,
                                     [&](int row, int m, float s, float) {
                                       __half* hp = a.h + (size_t)m * dim + row;
                                       *hp = hadd1(__ldcg(hp), __float2half_rn(s));
                                     },
                                     [&](int q, uint4 (&buf)[8]) { st_issue<R_D, NI_D, 1>(mn, q, buf, tid); });
      }
      if (!st_grid_sync(a, gen)) return;
    }

    // ================================================================== final norm -> logits, (value, lowest index) key
    stage_norm([&](int m) -> const __half* { return a.h + (size_t)m * dim; }, a.out_norm);
    {
      unsigned long long best = 0ull;
      const StepMat ml = mat(a.out_w, nullptr, a.vocab, KC_D);
      const bool again = step + 1 < a.n_steps;
      const StepMat m0 = mat(a.layers[0].wqkv, nullptr, qkv_dim, KC_D);
      st_project<R_D, NI_D, 1, MT>(ml, xs, dim, M, part, wv, tid,
                                   [&](int row, int m, float s, float) {
                                     const __half v = __float2half_rn(s);
                                     a.logits[(size_t)m * a.vocab + row] = v;
                                     const unsigned long long k = argmax_key(v, (uint32_t)row);
                                     best = k > best ? k : best;
                                   },
                                   [&](int q, uint4 (&buf)[8]) {
                                     if (again) st_issue<R_D, NI_D, 1>(m0, q, buf, tid);
                                   });
      if (warp == 0) {  // the finishing threads are tid < R_D * MT, row-major over (r, m)
#pragma unroll
        for (int m = 0; m < MT; m++) {
          unsigned long long v = (tid < R_D * MT && (tid % MT) == m) ? best : 0ull;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
            v = other > v ? other : v;
          }
          if (lane == 0 && m < M && v != 0ull) atomicMax(a.key + m, v);
        }
      }
    }
    if (!st_grid_sync(a, gen)) return;
    // every CTA reads the pick (the next step's embedding row); CTA 0 publishes it
#pragma unroll
    for (int m = 0; m < MT; m++) {
      if (m < M) {
        const unsigned long long k = __ldcg(a.key + m);
        tok[m] = (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
        if (bid == 0 && tid == 0) a.next_tokens[(size_t)step * M + m] = tok[m];
        if (a.advance) posv[m] += 1;
      }
    }
  }
  if (a.advance && bid == 0 && tid < M) {
#pragma unroll
    for (int m = 0; m < MT; m++)
      if (tid == m) { a.tokens[m] = tok[m]; a.pos[m] = posv[m]; }
  }
}

// ------------------------------------------------------------------------------------------------ host side
struct jg_step {
  jg_dev* dev;
  jg_kvcache* kv;
  StepArgs args;  // everything but the per-call buffers
  StepLayer* d_layers;
  int variant;    // index into the instantiation table
  int grid;
  int max_rows;
  size_t smem;
  int max_slices;
};

typedef void (*StepKernel)(const StepArgs);
struct StepVariant { int mt, hd, nrep, ni_d, ni_h; StepKernel kern; };
#define ST_VARIANT(MT, HD, NREP, NID, NIH) {MT, HD, NREP, NID, NIH, jg_step_kernel<MT, HD, NREP, NID, NIH>}
static const StepVariant g_step_variants[] = {
    ST_VARIANT(1, 128, 4, 1, 4), ST_VARIANT(2, 128, 4, 1, 4),  // Llama-3.1-8B: dim 4096, hidden 14336
    ST_VARIANT(1, 64, 4, 1, 2),  ST_VARIANT(2, 64, 4, 1, 2),   // Llama-3.2-1B: dim 2048, hidden 8192
    ST_VARIANT(1, 128, 3, 1, 2), ST_VARIANT(2, 128, 3, 1, 2),  // Llama-3.2-3B: dim 3072, hidden 8192
};

static int ni_for(int K) {  // chunk iterations per lane: the smallest of 1, 2, 4, 8 that covers K / 8 chunks with 512 lanes
  const int kc = K / 8;
  for (int ni = 1; ni <= 8; ni *= 2)
    if (kc <= ST_THREADS * ni) return ni;
  return 0;
}

static void step_destroy_now(void* p) {
  jg_step* s = (jg_step*)p;
  if (s->d_layers) cudaFree(s->d_layers);
  if (s->args.att_ml) cudaFree(s->args.att_ml);
  if (s->args.att_o) cudaFree(s->args.att_o);
  if (s->args.tickets) cudaFree(s->args.tickets);
  if (s->args.bar) cudaFree(s->args.bar);
  if (s->args.key) cudaFree(s->args.key);
  delete s;
}

JG_API int jg_step_create(jg_dev* dev, jg_kvcache* kv, const jg_step_desc* desc, jg_step** out) {
  JG_ENTER(dev);
  JG_REQUIRE(kv != nullptr && desc != nullptr && out != nullptr, "step_create: null argument");
  JG_REQUIRE(!dev->capturing, "step_create: not while a graph is being captured");
  const jg_step_desc& d = *desc;
  const jg_kvcache_desc& k = kv->d;
  JG_REQUIRE(d.n_layers > 0 && d.n_layers == k.n_layers && d.n_heads == k.n_heads && d.layers != 0, "step_create: layer / head counts do not match the cache");
  JG_REQUIRE(d.dim > 0 && d.hidden_dim > 0 && d.vocab_size > 0 && d.dim % 8 == 0 && d.hidden_dim % 8 == 0, "step_create: bad dimensions");
  JG_REQUIRE(jg_aligned(d.tok_embeddings, 16) && jg_aligned(d.out_norm, 16) && jg_aligned(d.output, 16) && jg_aligned(d.freqs_cis, 16) && d.freqs_rows > 0,
             "step_create: model tensors must be 16-byte aligned");
  const int nrep = k.n_heads / k.n_kv_heads;
  const int ni_d = ni_for(d.dim), ni_h = ni_for(d.hidden_dim);
  int variant = -1;
  const int nv = (int)(sizeof(g_step_variants) / sizeof(g_step_variants[0]));
  for (int i = 0; i < nv; i++)
    if (g_step_variants[i].mt == 1 && g_step_variants[i].hd == k.head_dim && g_step_variants[i].nrep == nrep &&
        g_step_variants[i].ni_d == ni_d && g_step_variants[i].ni_h == ni_h) { variant = i; break; }
  if (variant < 0 || k.n_heads * k.head_dim != d.dim) {
    jg_set_error("step_create: no single-kernel step for dim %d, hidden %d, head_dim %d, %d query heads per kv head", d.dim, d.hidden_dim, k.head_dim, nrep);
    return JG_ENOTSUP;
  }
  const int max_rows = 2;
  const int grid = dev->sm_count;
  JG_REQUIRE(grid >= max_rows * k.n_kv_heads, "step_create: fewer SMs than (row, kv head) pairs");
  // context slices per (row, kv head): as many as the CTAs allow (at most 32); one slice's scores must fit
  const int slices_min = grid / (max_rows * k.n_kv_heads) < 32 ? grid / (max_rows * k.n_kv_heads) : 32;
  const int chunk_cap = ((kv->max_ctx + slices_min - 1) / slices_min + 31) & ~31;
  const size_t att_bytes = ((size_t)nrep * chunk_cap + (size_t)ST_WARPS * nrep * k.head_dim + (size_t)nrep * k.head_dim) * sizeof(float);
  const size_t x_bytes = (size_t)max_rows * (d.dim > d.hidden_dim ? d.dim : d.hidden_dim) * sizeof(__half);
  const size_t smem = att_bytes > x_bytes ? att_bytes : x_bytes;
  if (smem + 8 * 1024 > (size_t)dev->prop.sharedMemPerBlockOptin) {
    jg_set_error("step_create: %zu bytes of shared memory per CTA needed, the device allows %zu", smem, (size_t)dev->prop.sharedMemPerBlockOptin);
    return JG_ENOTSUP;
  }
  int coop = 0;
  JG_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev->ordinal));
  if (!coop) { jg_set_error("step_create: the device does not support cooperative launches"); return JG_ENOTSUP; }
  for (int i = variant; i < variant + 2; i++) {
    JG_CUDA(cudaFuncSetAttribute(g_step_variants[i].kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, g_step_variants[i].kern, ST_THREADS, smem));
    if (per_sm < 1) { jg_set_error("step_create: the step kernel does not fit an SM"); return JG_ENOTSUP; }
  }
  jg_step* s = new jg_step();
  memset(s, 0, sizeof(*s));
  s->dev = dev; s->kv = kv; s->variant = variant; s->grid = grid; s->max_rows = max_rows; s->smem = smem; s->max_slices = 32;
  StepArgs& a = s->args;
  a.tok_emb = (const __half*)d.tok_embeddings; a.out_norm = (const __half*)d.out_norm; a.out_w = (const __half*)d.output;
  a.table = (const __half*)d.freqs_cis; a.table_rows = d.freqs_rows;
  a.k_pool = kv->k_pool; a.v_pool = kv->v_pool; a.block_table = kv->block_table; a.layer_elems = kv->layer_elems;
  a.n_layers = d.n_layers; a.dim = d.dim; a.hidden = d.hidden_dim; a.H = k.n_heads; a.G = k.n_kv_heads; a.vocab = d.vocab_size;
  a.page = k.page_size; a.page_shift = ilog2(k.page_size); a.max_pages_per_seq = k.max_pages_per_seq; a.max_ctx = kv->max_ctx;
  a.chunk_cap = chunk_cap;
  a.eps = d.norm_eps; a.scale = 1.0f / sqrtf((float)k.head_dim); a.recip_dim = 1.0f / (float)d.dim;
  const char* te = getenv("JG_STEP_TIMEOUT_MS");
  a.timeout_ns = (unsigned long long)(te ? atoll(te) : 2000) * 1000000ull;
  const char* ge = getenv("JG_STEP_L2_ROWS");
  a.l2_gu_rows = ge ? atoi(ge) : 16;
  // the layers' tensors, as a device table
  const uint64_t* lp = (const uint64_t*)(uintptr_t)d.layers;
  StepLayer* hl = new StepLayer[d.n_layers];
  bool ok = true;
  for (int l = 0; l < d.n_layers; l++) {
    for (int j = 0; j < 7; j++) ok = ok && jg_aligned(lp[l * 7 + j], 16);
    hl[l].attn_norm = (const __half*)lp[l * 7 + 0]; hl[l].wqkv = (const __half*)lp[l * 7 + 1]; hl[l].wo = (const __half*)lp[l * 7 + 2];
    hl[l].ffn_norm = (const __half*)lp[l * 7 + 3]; hl[l].w1 = (const __half*)lp[l * 7 + 4]; hl[l].w3 = (const __half*)lp[l * 7 + 5];
    hl[l].w2 = (const __half*)lp[l * 7 + 6];
  }
  cudaError_t e = ok ? cudaSuccess : cudaErrorInvalidValue;
  const size_t pairs = (size_t)max_rows * k.n_kv_heads;
  if (e == cudaSuccess) e = cudaMalloc(&s->d_layers, sizeof(StepLayer) * d.n_layers);
  if (e == cudaSuccess) e = cudaMemcpyAsync(s->d_layers, hl, sizeof(StepLayer) * d.n_layers, cudaMemcpyHostToDevice, dev->stream);
  if (e == cudaSuccess) e = cudaMalloc(&a.att_ml, pairs * nrep * 32 * 2 * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&a.att_o, pairs * 32 * nrep * k.head_dim * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&a.tickets, pairs * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMalloc(&a.bar, 64 * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMalloc(&a.key, 2 * sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMemsetAsync(a.tickets, 0, pairs * sizeof(unsigned int), dev->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(a.bar, 0, 64 * sizeof(unsigned int), dev->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
  delete[] hl;
  if (e != cudaSuccess) {
    step_destroy_now(s);
    if (!ok) { jg_set_error("step_create: a layer tensor is null or not 16-byte aligned"); return JG_EINVAL; }
    return jg_cuda_fail(e, "step_create", __FILE__, __LINE__);
  }
  a.layers = s->d_layers;
  if (dev->err_word == nullptr) {
    JG_CUDA(cudaMalloc(&dev->err_word, sizeof(int)));
    JG_CUDA(cudaMemset(dev->err_word, 0, sizeof(int)));
  }
  a.err = dev->err_word;
  *out = s;
  return JG_OK;
}

JG_API int jg_step_destroy(jg_step* s) {
  if (s == nullptr) return JG_OK;
  if (g_jg_capturing > 0) { jg_defer(step_destroy_now, s); return JG_OK; }
  cudaSetDevice(s->dev->ordinal);
  cudaStreamSynchronize(s->dev->stream);
  step_destroy_now(s);
  return JG_OK;
}

JG_API int jg_step_run(jg_step* s, uint64_t tokens, uint64_t pos, uint64_t h, uint64_t qkv, uint64_t attn, uint64_t ffn,
                       uint64_t logits, uint64_t next_tokens, int32_t B, int32_t n_steps, int32_t advance) {
  JG_REQUIRE(s != nullptr, "step_run: null handle");
  jg_dev* dev = s->dev;
  JG_ENTER(dev);
  JG_REQUIRE(B >= 1 && B <= s->max_rows && B <= s->kv->d.max_batch, "step_run: %d rows (1..%d)", B, s->max_rows);
  JG_REQUIRE(n_steps >= 1 && (n_steps == 1 || advance), "step_run: several steps only with advance");
  JG_REQUIRE(jg_aligned(tokens, 4) && jg_aligned(pos, 4) && jg_aligned(next_tokens, 4), "step_run: token / position buffers");
  JG_REQUIRE(jg_aligned(h, 16) && jg_aligned(qkv, 16) && jg_aligned(attn, 16) && jg_aligned(ffn, 16) && jg_aligned(logits, 16), "step_run: activation buffers must be 16-byte aligned");
  StepArgs a = s->args;
  a.tokens = (int32_t*)tokens; a.pos = (int32_t*)pos; a.next_tokens = (int32_t*)next_tokens;
  a.h = (__half*)h; a.qkv = (__half*)qkv; a.attn = (__half*)attn; a.ffn = (__half*)ffn; a.logits = (__half*)logits;
  a.M = B; a.n_steps = n_steps; a.advance = advance ? 1 : 0;
  int sl = s->grid / (B * a.G);
  if (sl > s->max_slices) sl = s->max_slices;
  a.slices = sl;
  JG_REQUIRE((long long)sl * a.chunk_cap >= a.max_ctx, "step_run: context slices do not cover the cache");
  const StepVariant& v = g_step_variants[s->variant + (B > 1 ? 1 : 0)];
  // the arrival count starts at zero whatever an earlier launch that ran out of time left behind
  JG_CUDA(cudaMemsetAsync(a.bar, 0, sizeof(unsigned int), dev->stream));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(s->grid);
  cfg.blockDim = dim3(ST_THREADS);
  cfg.dynamicSmemBytes = s->smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, v.kern, (const StepArgs)a);
  if (e != cudaSuccess) return jg_cuda_fail(e, "step", __FILE__, __LINE__);
  dev->tc_pending = true;  // the error word is looked at after the next synchronisation
  return jg_after_launch(dev, "step");
}
