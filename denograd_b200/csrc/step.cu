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
#include <stdio.h>

#include "common.cuh"
#include "kvcache.cuh"
#include "peer.cuh"
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
  int slices, chunk_cap;  // most context slices per (row, kv head) and the scores one slice can hold
  int slice_len;          // positions a slice aims at
  int advance, n_steps;
  int nslot;        // slots of the weight ring (passes in flight per CTA)
  int q_dim;        // H * head_dim: columns of Wo (a rank's share of the heads under tensor parallelism)
  int embed_rows;   // rows of the embedding table (the whole vocabulary on every rank)
  int vocab_offset; // vocabulary index of row 0 of this rank's output matrix
  uint32_t peer_ord0;  // tensor parallelism: ordinal of the launch's first exchange (peer.ord is not used)
  int bar_probe;    // JG_STEP_PROF=2: that many back-to-back grid barriers at the start of every launch, timed in slot 15
  int slot_bytes;   // bytes of one slot = of one pass: a few whole rows of one matrix (or of the gate / up pair)
  int ring_offset;  // bytes from the start of dynamic shared memory to the ring
  unsigned long long* prof;  // JG_STEP_PROF=1: [2][16] nanoseconds per phase, summed over layers and steps (CTA 0, last CTA)
  float eps, scale, recip_dim;
  PeerArgs peer;  // tensor parallelism (peer.world > 1): the ranks' exchange buffers, as in the stand-alone projections
};

constexpr int ST_MAX_SLOTS = 6;

__device__ __forceinline__ unsigned long long st_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_cg_128(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t st_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Bounded wait for the phase of `bar` with the given parity (a bulk copy's bytes have landed); false = gave up.
__device__ __forceinline__ bool st_mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long timeout_ns) {
  const uint32_t addr = st_smem_u32(bar);
  unsigned long long t0 = 0;
  for (unsigned polls = 1;; polls++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((polls & 63u) == 0) {
      const unsigned long long now = st_now();
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) return false;
    }
  }
}

// Grid-wide barrier: every CTA adds one to a counter the host zeroed before the launch and waits until the counter
// reaches the barrier's ordinal times the grid size.  All CTAs are resident (cooperative launch).  Returns false when
// the wait ran out; the caller leaves the kernel.
__device__ __forceinline__ bool st_grid_sync(const StepArgs& a, unsigned& nbar) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    nbar++;
    const unsigned target = nbar * gridDim.x;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.bar) : "memory");
    // (several polls in flight per CTA were measured: two change nothing, four slow the counter's line down: 1.44 -> 2.26 us)
    unsigned long long t0 = 0;
    for (unsigned polls = 1;; polls++) {
      unsigned v;
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.bar) : "memory");
      if (v >= target) break;
      if ((polls & 255u) == 0) {
        const unsigned long long now = st_now();
        if (t0 == 0) t0 = now;
        else if (now - t0 > a.timeout_ns) { ok = 0; break; }
      }
    }
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
    s_ok = ok;
    if (!ok) atomicCAS(a.err, 0, 4);
  }
  __syncthreads();
  return s_ok != 0;
}

// ---- the weight stream.  Thread 0 of the CTA walks the step's projections in order (qkv, wo, gate/up, down of every
// layer, then the output matrix, then the next step) and keeps `nslot` passes in flight as bulk copies into a ring of
// shared-memory slots; the copy of pass q + nslot is issued the moment pass q has been consumed.  The walk does not stop
// at phase boundaries: while the CTA stages activations, waits at a grid barrier or works on attention, the first
// passes of the next projection are landing.
// How an N-row matrix is dealt to the CTAs in passes of rs rows: CTA c takes passes c, c + grid, c + 2 grid, ... (at
// any moment the grid reads one contiguous window of the matrix); the matrix's last pass may be short.  (Splitting the
// rows that do not fill a whole round evenly over the CTAs was measured and is slower: every CTA then pays a pass's
// fixed cost for a few rows.)
struct StepSplit { int passes, last_rows; };  // passes of this CTA; rows of its last pass
__device__ __forceinline__ StepSplit st_split(int N, int rs) {
  const int bid = blockIdx.x, nb = gridDim.x;
  const int total = (N + rs - 1) / rs;
  StepSplit sp;
  sp.passes = bid < total ? (total - bid + nb - 1) / nb : 0;
  const bool short_last = sp.passes > 0 && bid + (sp.passes - 1) * nb == total - 1;
  sp.last_rows = short_last ? N - (total - 1) * rs : rs;
  return sp;
}

struct StepStream {
  int step, layer, phase;  // phase: 0 qkv, 1 wo, 2 gate/up, 3 down, 4 output matrix; step == n_steps: nothing left
  int left;                // passes this CTA still has to request in the phase
  uint32_t pass_bytes;     // bytes of a full pass (per matrix), of this CTA's last pass of the phase
  uint32_t tail_bytes;
  const unsigned char* src0;  // next pass of the first (second) matrix
  const unsigned char* src1;
  uint32_t slot;           // ring slot the next pass goes to
  size_t stride;           // bytes from one pass of this CTA to its next
};

// Position (step, layer, phase) -> matrix, this CTA's rows, passes (0 when the CTA has no rows in the phase).
template <int RS_D, int RS_G, int RS_H>
__device__ __forceinline__ void st_stream_enter(StepStream& st, const StepArgs& a, int qkv_dim) {
  const int bid = blockIdx.x, nb = gridDim.x;
  int N, rs;
  const StepLayer* L = a.layers + st.layer;
  const unsigned char* w0;
  const unsigned char* w1 = nullptr;
  uint32_t row_bytes = (uint32_t)a.dim * 2u;
  switch (st.phase) {
    case 0: N = qkv_dim; rs = RS_D; w0 = reinterpret_cast<const unsigned char*>(L->wqkv); break;
    case 1: N = a.dim; rs = RS_D; w0 = reinterpret_cast<const unsigned char*>(L->wo); row_bytes = (uint32_t)a.q_dim * 2u; break;
    case 2: N = a.hidden; rs = RS_G; w0 = reinterpret_cast<const unsigned char*>(L->w1); w1 = reinterpret_cast<const unsigned char*>(L->w3); break;
    case 3: N = a.dim; rs = RS_H; w0 = reinterpret_cast<const unsigned char*>(L->w2); row_bytes = (uint32_t)a.hidden * 2u; break;
    default: N = a.vocab; rs = RS_D; w0 = reinterpret_cast<const unsigned char*>(a.out_w); break;
  }
  const StepSplit sp = st_split(N, rs);
  st.left = sp.passes;
  st.pass_bytes = (uint32_t)rs * row_bytes;
  st.stride = (size_t)nb * st.pass_bytes;
  st.tail_bytes = (uint32_t)sp.last_rows * row_bytes;
  st.src0 = w0 + (size_t)bid * st.pass_bytes;
  st.src1 = w1 ? w1 + (size_t)bid * st.pass_bytes : nullptr;
}
template <int RS_D, int RS_G, int RS_H>
__device__ __forceinline__ void st_stream_next_phase(StepStream& st, const StepArgs& a, int qkv_dim) {
  do {
    if (st.phase == 4) { st.phase = 0; st.layer = 0; st.step++; }
    else if (st.phase == 3) { st.layer++; st.phase = (st.layer < a.n_layers) ? 0 : 4; if (st.phase == 4) st.layer = 0; }
    else st.phase++;
    if (st.step >= a.n_steps) return;
    st_stream_enter<RS_D, RS_G, RS_H>(st, a, qkv_dim);
  } while (st.left <= 0);
}
// Request the next pass of the walk into the slot that has just been consumed (the CTA's producer thread only).
template <int RS_D, int RS_G, int RS_H>
__device__ __forceinline__ void st_stream_issue(StepStream& st, const StepArgs& a, int qkv_dim, unsigned char* ring, uint64_t* full) {
  if (st.step >= a.n_steps) return;
  const uint32_t bytes = st.left == 1 ? st.tail_bytes : st.pass_bytes;
  const unsigned char* s0 = st.src0;
  const unsigned char* s1 = st.src1;
  const uint32_t bar = st_smem_u32(full + st.slot);
  const uint32_t dst = st_smem_u32(ring) + st.slot * (uint32_t)a.slot_bytes;
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(st.src1 ? 2u * bytes : bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(s0), "r"(bytes), "r"(bar) : "memory");
  if (st.src1) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst + st.pass_bytes), "l"(s1), "r"(bytes), "r"(bar) : "memory");
    st.src1 += st.stride;
  }
  st.src0 += st.stride;
  st.slot = (st.slot + 1 == (uint32_t)a.nslot) ? 0u : st.slot + 1;
  if (--st.left == 0) st_stream_next_phase<RS_D, RS_G, RS_H>(st, a, qkv_dim);
}

// Where the consumer is in the ring: slot of the next pass and the parity of that slot's barrier.
struct StepRing { uint32_t slot, parity; };

constexpr int ST_PRODUCER = ST_THREADS - 32;  // the thread that requests the weight passes (lane 0 of the last warp)

// One projection phase of this CTA: its passes of RS rows (of each of NW matrices) of an N-row matrix; thread t multiplies
// the 16-byte chunks t, t + 512, ... of every row of the pass (read from the slot) with the activations; the per-warp
// partial sums meet in shared memory at one barrier per pass, after which the producer thread refills the slot and
// output o of the pass (o < RS * MT) is finished by lane 0 of warp o, in warp order (fixed summation order) — one
// output per warp, so that no warp carries the whole epilogue.  `pre(row, m)` fetches what the epilogue needs from
// global memory (the residual) before the pass is multiplied.  A data wait that runs out is recorded and the pass is
// carried on with whatever the slot holds (the launch's results are void then).
template <int RS, int NI, int NW, int MT, class Pre, class Epi, class Refill>
__device__ __forceinline__ void st_project(int N, int KC, const __half* xs, int M, const unsigned char* ring, uint64_t* full,
                                           StepRing& rg, unsigned& seq, float (*part)[ST_PART * ST_WARPS], const StepArgs& a, int tid,
                                           Pre pre, Epi epi, Refill refill) {
  static_assert(RS * NW * MT <= ST_PART && RS * MT <= ST_WARPS, "partial sums per warp; one output per finishing warp");
  const int K = KC * 8;
  const uint32_t row_bytes = (uint32_t)KC * 16u;
  const int bid = blockIdx.x, nb = gridDim.x;
  const StepSplit sp = st_split(N, RS);
  const int np = sp.passes;
  const int lane = tid & 31, warp = tid >> 5;
  const int fr = warp / MT, fm = warp % MT;  // the output lane 0 of this warp finishes (warp < RS * MT)
  for (int p = 0; p < np; p++) {
    const int frow = (bid + p * nb) * RS + fr;
    const bool fin = lane == 0 && warp < RS * MT && fm < M && frow < N;
    __half prev = __float2half_rn(0.f);
    if (fin) prev = pre(frow, fm);
    if (!st_mbar_wait(full + rg.slot, rg.parity, a.timeout_ns)) atomicCAS(a.err, 0, 5);
    const unsigned char* sl = ring + (size_t)rg.slot * a.slot_bytes;
    float acc[NW * RS][MT];
#pragma unroll
    for (int j = 0; j < NW * RS; j++)
#pragma unroll
      for (int m = 0; m < MT; m++) acc[j][m] = 0.f;
#pragma unroll
    for (int i = 0; i < NI; i++) {
      const int c = tid + ST_THREADS * i;
      if (c < KC) {
        float xf[MT][8];
#pragma unroll
        for (int m = 0; m < MT; m++) unpack8(*reinterpret_cast<const uint4*>(xs + (size_t)m * K + (size_t)c * 8), xf[m]);
#pragma unroll
        for (int j = 0; j < NW * RS; j++) {
          const uint4 wv = *reinterpret_cast<const uint4*>(sl + (size_t)j * row_bytes + (size_t)c * 16);
#pragma unroll
          for (int m = 0; m < MT; m++) acc[j][m] = dot8_acc(acc[j][m], wv, xf[m]);
        }
      }
    }
    float* pp = part[seq & 1u];  // [value][warp]
#pragma unroll
    for (int j = 0; j < NW * RS; j++)
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const float v = warp_sum(acc[j][m]);
        if (lane == 0) pp[(j * MT + m) * ST_WARPS + warp] = v;
      }
    __syncthreads();
    if (tid == ST_PRODUCER) refill();
    if (fin) {
      auto sum16 = [&](int value) {
        const float4* q = reinterpret_cast<const float4*>(pp + value * ST_WARPS);
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < ST_WARPS / 4; w++) {
          const float4 v = q[w];
          t += v.x; t += v.y; t += v.z; t += v.w;
        }
        return t;
      };
      const float s_a = sum16(fr * MT + fm);
      const float s_b = NW == 2 ? sum16((RS + fr) * MT + fm) : 0.f;
      epi(frow, fm, s_a, s_b, prev);
    }
    seq++;
    if (++rg.slot == (uint32_t)a.nslot) { rg.slot = 0; rg.parity ^= 1u; }
  }
}

// RS_D / RS_G / RS_H: rows per pass of a projection with K = dim (one matrix), of the gate / up pair (rows of each), with
// K = hidden; NI_D / NI_H: 16-byte chunks per thread and row (K / 8 chunks over 512 threads).
template <int MT, int HD, int NREP, int RS_D, int RS_G, int RS_H, int NI_D, int NI_H>
__global__ void __launch_bounds__(ST_THREADS, 1) jg_step_kernel(const StepArgs a) {
  static_assert(NREP <= 4 && MT <= 2, "register budget of 128 per thread");
  constexpr int LPR = HD / 8;    // lanes per K / V row
  constexpr int RPW = 32 / LPR;  // rows per warp pass
  constexpr int AU = 2;          // attention row passes in flight
  constexpr int ROWS_IT = ST_WARPS * RPW * AU;

  extern __shared__ __align__(16) unsigned char st_smem[];
  __half* xs = reinterpret_cast<__half*>(st_smem);  // [MT][K] activation rows of a projection phase
  // the attention phases reuse the same bytes: raw scores, per-warp p.v partials, the CTA's p.v partial
  float* sc = reinterpret_cast<float*>(st_smem);                     // [NREP][chunk_cap]
  float* pv_part = sc + (size_t)NREP * a.chunk_cap;                   // [ST_WARPS / 2][NREP][HD]
  unsigned char* ring = st_smem + a.ring_offset;                     // [nslot][slot_bytes] weight passes in flight
  __shared__ __align__(8) uint64_t full[ST_MAX_SLOTS];
  __shared__ __align__(16) float part[2][ST_PART * ST_WARPS];
  __shared__ float red[ST_WARPS][4];
  __shared__ float s_rs[MT];
  __shared__ float s_m[4], s_M[4], s_rL[4];
  __shared__ int s_last;
  __shared__ unsigned long long s_key[MT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bid = blockIdx.x, nb = gridDim.x;
  const int dim = a.dim, hidden = a.hidden, M = a.M;
  const int KC_D = dim / 8, KC_H = hidden / 8, KC_Q = a.q_dim / 8;
  // tensor parallelism: Wo and W2 hold this rank's columns only, so their outputs are partial sums.  Each is sent to every
  // rank (this one included) as a flag-in-data entry the moment it is complete; when the CTA has multiplied its last
  // pass of the phase it collects, for the outputs it owns, the entries of all ranks (bounded wait), adds them in rank
  // order and applies the residual.  Exchange k of the launch carries the number base + k; consecutive exchanges
  // alternate between the two halves of the buffers, and the grid barrier after a phase keeps a rank from starting
  // exchange k + 1 before all of its CTAs have read exchange k - 1.
  const int world = a.peer.world > 1 ? a.peer.world : 1;
  const uint32_t peer_base = world > 1 ? a.peer.epoch[0] + a.peer_ord0 : 0u;
  const int qkv_dim = (a.H + 2 * a.G) * HD;
  const float log2e = 1.4426950408889634f;

  unsigned gen = 0;  // grid barriers passed
  unsigned seq = 0;  // weight passes consumed

  // the weight stream starts before anything else: nslot passes are on their way while the first rows are staged
  StepStream st;
  StepRing rg;
  rg.slot = 0; rg.parity = 0;
  unsigned issued = 0;  // passes requested (producer thread)
  if (tid == ST_PRODUCER) {
    for (int i = 0; i < a.nslot; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(st_smem_u32(full + i)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    st.step = 0; st.layer = 0; st.phase = 0; st.slot = 0;
    st_stream_enter<RS_D, RS_G, RS_H>(st, a, qkv_dim);
    if (st.left <= 0) st_stream_next_phase<RS_D, RS_G, RS_H>(st, a, qkv_dim);
    for (int i = 0; i < a.nslot; i++) {
      if (st.step < a.n_steps) issued++;
      st_stream_issue<RS_D, RS_G, RS_H>(st, a, qkv_dim, ring, full);
    }
  }
  __syncthreads();
  auto refill = [&]() {
    if (st.step < a.n_steps) issued++;
    st_stream_issue<RS_D, RS_G, RS_H>(st, a, qkv_dim, ring, full);
  };
  auto no_pre = [](int, int) { return __float2half_rn(0.f); };
  auto residual = [&](int row, int m) { return __ldcg(a.h + (size_t)m * dim + row); };
  const uint32_t ex_per_step = (uint32_t)(2 * a.n_layers + 1);  // exchanges of a step: Wo and W2 of every layer, the pick
  // output (row, m) of a row-parallel projection: the residual add on one GPU, an entry for every rank otherwise
  auto rowpar_epi = [&](uint32_t ex, int row, int m, float sum, __half prev) {
    const size_t o = (size_t)m * dim + row;
    if (world == 1) {
      a.h[o] = hadd1(prev, __float2half_rn(sum));
      return;
    }
    for (int p = 0; p < world; p++) peer_ll_store(peer_ll(a.peer.buf[p], (int)(ex & 1u), a.peer.rank) + o, sum, ex);
  };
  // after the phase's last pass: the outputs this CTA owns (its passes of rs rows) summed over the ranks in rank order
  auto rowpar_gather = [&](uint32_t ex, int rs) {
    if (world == 1) return;
    const int total = (dim + rs - 1) / rs;
    const int np = bid < total ? (total - bid + nb - 1) / nb : 0;
    bool ok = true;
    for (int i = tid; i < np * rs * M; i += ST_THREADS) {
      const int m = i % M, rr = i / M;
      const int row = (bid + (rr / rs) * nb) * rs + rr % rs;
      if (row < dim) {
        const size_t o = (size_t)m * dim + row;
        // the ranks' entries are requested together (one round trip to this GPU's memory for all of them); an entry
        // that has not arrived yet is polled, bounded
        uint32_t val[PEER_MAX_WORLD], tag[PEER_MAX_WORLD];
        const __half h_old = __ldcg(a.h + o);
#pragma unroll
        for (int rk = 0; rk < PEER_MAX_WORLD; rk++) {
          val[rk] = 0u;
          tag[rk] = ex;
          if (rk < world)
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(val[rk]), "=r"(tag[rk])
                         : "l"(peer_ll(a.peer.buf[a.peer.rank], (int)(ex & 1u), rk) + o) : "memory");
        }
        float sum = 0.f;
#pragma unroll
        for (int rk = 0; rk < PEER_MAX_WORLD; rk++) {
          if (rk < world) {
            float v = __uint_as_float(val[rk]);
            if (tag[rk] != ex && ok) ok = peer_ll_load(peer_ll(a.peer.buf[a.peer.rank], (int)(ex & 1u), rk) + o, ex, a.peer.timeout_ns, &v);
            sum = __fadd_rn(sum, v);
          }
        }
        a.h[o] = hadd1(h_old, __float2half_rn(sum));
      }
    }
    if (!ok) atomicCAS(a.peer.err, 0, 1);  // a rank never arrived: the launch's results are void, nobody is waited for
  };
  // a wait ran out: record it, let the copies still in flight land (bounded) so that none writes into shared memory of
  // a CTA that has gone, and leave
  auto give_up = [&](int code) {
    if (tid == ST_PRODUCER) {
      atomicCAS(a.err, 0, code);
      StepRing r = rg;
      for (unsigned q = seq; q < issued; q++) {
        st_mbar_wait(full + r.slot, r.parity, a.timeout_ns);
        if (++r.slot == (uint32_t)a.nslot) { r.slot = 0; r.parity ^= 1u; }
      }
    }
    __syncthreads();
  };

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

  // phase timing (diagnostic): CTA 0 and the last CTA add the time since their previous stamp to slot `i`
  unsigned long long t_prev = 0;
  const bool prof = a.prof != nullptr && tid == 0 && (bid == 0 || bid == nb - 1);
  if (prof) {
    t_prev = st_now();
    if (bid == 0) { a.prof[14] += 1ull; a.prof[30] += (unsigned long long)a.n_steps; }  // launches and steps, replays included
  }
  auto stamp = [&](int i) {
    if (prof) {
      const unsigned long long t = st_now();
      a.prof[(bid == 0 ? 0 : 16) + i] += t - t_prev;
      t_prev = t;
    }
  };

  if (a.prof != nullptr && a.bar_probe > 0) {  // diagnostic: the cost of a grid barrier nobody arrives late at
    for (int i = 0; i < a.bar_probe; i++)
      if (!st_grid_sync(a, gen)) { give_up(4); return; }
    stamp(15);
  }
  for (int step = 0; step < a.n_steps; step++) {
    for (int l = 0; l < a.n_layers; l++) {
      const StepLayer* L = a.layers + l;
      // this CTA's share of attention: context slice `slice` of (row b, kv head g); the pages of its first rows are looked
      // up now, so that the rows themselves can be requested without a dependent load when the projection is over
      const int n_pairs = M * a.G;
      const bool mine = bid < n_pairs * a.slices;  // a.slices: the most slices a pair can have (the scratch's stride)
      const int pair = mine ? bid / a.slices : 0, slice = mine ? bid % a.slices : 0;
      const int b = pair / a.G, g = pair % a.G;
      const int sub = lane % LPR, rgrp = lane / LPR;
      int pb = posv[0];
#pragma unroll
      for (int m = 1; m < MT; m++) pb = (b == m) ? posv[m] : pb;
      const int T = min(max(pb + 1, 1), a.max_ctx);
      const int pnew = T - 1;
      // slices of this pair: about a.slice_len positions each (a short context keeps few CTAs busy and the exchanges of
      // statistics and partials short), never more positions than a slice's scores have room for
      const int S = min(a.slices, max((T + a.slice_len - 1) / a.slice_len, (T + a.chunk_cap - 1) / a.chunk_cap));
      const bool att = mine && slice < S;
      const int chunk = (T + S - 1) / S;
      const int t0 = slice * chunk, t1 = att ? min(T, t0 + chunk) : t0;
      const int32_t* bt_row = a.block_table + (size_t)b * a.max_pages_per_seq;
      __half* k_layer = a.k_pool + (size_t)l * a.layer_elems;
      __half* v_layer = a.v_pool + (size_t)l * a.layer_elems;
      int pg0[AU];
#pragma unroll
      for (int u = 0; u < AU; u++) {
        const int t = t0 + warp * RPW + rgrp + u * ST_WARPS * RPW;
        pg0[u] = (att && t < t1) ? bt_row[t >> a.page_shift] : 0;
      }
      // ================================================================ P1: norm -> qkv
      if (l == 0) {
        // the embedding rows are the block's input (a token outside the table matches no row: zeros); CTA 0 stores them
        // as the residual stream
        auto emb = [&](int m) -> const __half* {
          return ((unsigned)tok[m] < (unsigned)a.embed_rows) ? a.tok_emb + (size_t)tok[m] * dim : nullptr;
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
      st_project<RS_D, NI_D, 1, MT>(qkv_dim, KC_D, xs, M, ring, full, rg, seq, part, a, tid, no_pre,
                                         [&](int row, int m, float s, float, __half) { a.qkv[(size_t)m * qkv_dim + row] = __float2half_rn(s); },
                                         refill);
      // the first K and V rows of this CTA's context slice are requested now, ahead of the barrier: cached rows do not
      // depend on this step's projection (the new position's row does and is fetched again once it has been written)
      uint4 k0[AU], v0[AU];
#pragma unroll
      for (int u = 0; u < AU; u++) {
        const int t = t0 + warp * RPW + rgrp + u * ST_WARPS * RPW;
        const bool ld = att && t < t1 && t != pnew;
        const size_t off = (((size_t)pg0[u] * a.G + g) * a.page + (t & (a.page - 1))) * HD + sub * 8;
        k0[u] = ld ? ld_cg_128(k_layer + off) : make_uint4(0, 0, 0, 0);
        v0[u] = ld ? ld_cg_128(v_layer + off) : make_uint4(0, 0, 0, 0);
      }
      stamp(0);
      if (!st_grid_sync(a, gen)) { give_up(4); return; }
      stamp(1);
      if (l == 0 && bid == 0 && tid < M) a.key[tid] = 0ull;  // every CTA has read the previous step's key by now

      // ================================================================ P2: RoPE, cache write, scores of a context slice
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
            if (base == t0 && t != pnew) {
              kk[u] = k0[u];  // requested before the barrier
            } else {
              kk[u] = (t < t1) ? ld_cg_128(kv_row(k_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
              if (base == t0) v0[u] = (t < t1) ? ld_cg_128(kv_row(v_layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + sub * 8) : make_uint4(0, 0, 0, 0);
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
      stamp(2);
      if (!st_grid_sync(a, gen)) { give_up(4); return; }
      stamp(3);

      // ================================================================ P3: probabilities, p.v, fold over the slices
      if (att) {
        // every (head, slice) pair of statistics is fetched by its own thread (one round trip to L2 for all of them), then
        // one thread per head combines them in slice order
        float* ml_s = pv_part;  // [NREP][slices][2], free until the p.v partials are stored
        if (tid < NREP * S) {
          const int r = tid / S, j = tid % S;
          const float2 v = __ldcg(reinterpret_cast<const float2*>(a.att_ml + (((size_t)pair * NREP + r) * a.slices + j) * 2));
          ml_s[2 * tid] = v.x;
          ml_s[2 * tid + 1] = v.y;
        }
        __syncthreads();
        if (tid < NREP) {
          const float* ml = ml_s + (size_t)tid * S * 2;
          float Mx = -INFINITY;
          for (int j = 0; j < S; j++) Mx = fmaxf(Mx, ml[2 * j]);
          float Ls = 0.f;
          for (int j = 0; j < S; j++)
            Ls = __fadd_rn(Ls, __fmul_rn(ml[2 * j + 1], jg_xexp2_f32(__fmul_rn(__fsub_rn(ml[2 * j], Mx), log2e))));
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
        // the warps' partials meet in two rounds (upper half of the warps stores, lower half adds its own on top), which
        // halves the scratch
        if (rgrp == 0 && warp >= ST_WARPS / 2) {
#pragma unroll
          for (int r = 0; r < NREP; r++)
#pragma unroll
            for (int i = 0; i < 8; i++) pv_part[((size_t)(warp - ST_WARPS / 2) * NREP + r) * HD + sub * 8 + i] = acc[r][i];
        }
        __syncthreads();
        if (rgrp == 0 && warp < ST_WARPS / 2) {
#pragma unroll
          for (int r = 0; r < NREP; r++)
#pragma unroll
            for (int i = 0; i < 8; i++) pv_part[((size_t)warp * NREP + r) * HD + sub * 8 + i] += acc[r][i];
        }
        __syncthreads();
        float* po = a.att_o + ((size_t)pair * a.slices + slice) * (NREP * HD);
        for (int idx = tid; idx < NREP * HD; idx += ST_THREADS) {
          float s = 0.f;
#pragma unroll
          for (int w = 0; w < ST_WARPS / 2; w++) s += pv_part[(size_t)w * NREP * HD + idx];
          po[idx] = s;
        }
        // the last CTA of the pair to get here folds the slices in slice order (the ticket's release covers the whole
        // CTA's stores: they are ordered before it by the barrier)
        __syncthreads();
        if (tid == 0) {
          unsigned prev;
          asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(a.tickets + pair) : "memory");
          s_last = (prev == (unsigned)S - 1u);
          if (s_last) a.tickets[pair] = 0;
          __threadfence();
        }
        __syncthreads();
        if (s_last) {
          const float* pall = a.att_o + (size_t)pair * a.slices * (NREP * HD);
          for (int idx = tid; idx < NREP * HD; idx += ST_THREADS) {
            float s = 0.f;
            for (int j0 = 0; j0 < S; j0 += 8) {  // eight slices' values requested together, added in slice order
              float v[8];
#pragma unroll
              for (int jj = 0; jj < 8; jj++) v[jj] = (j0 + jj < S) ? __ldcg(pall + (size_t)(j0 + jj) * (NREP * HD) + idx) : 0.f;
#pragma unroll
              for (int jj = 0; jj < 8; jj++)
                if (j0 + jj < S) s = __fadd_rn(s, v[jj]);
            }
            a.attn[(size_t)b * a.H * HD + (size_t)g * NREP * HD + idx] = __float2half_rn(s);
          }
        }
      }
      stamp(4);
      if (!st_grid_sync(a, gen)) { give_up(4); return; }
      stamp(5);

      // ================================================================ P4: h += Wo attn
      stage_copy(a.attn, a.q_dim);
      {
        const uint32_t ex = peer_base + (uint32_t)step * ex_per_step + 2u * (uint32_t)l;
        st_project<RS_D, NI_D, 1, MT>(dim, KC_Q, xs, M, ring, full, rg, seq, part, a, tid, residual,
                                      [&](int row, int m, float s, float, __half prev) { rowpar_epi(ex, row, m, s, prev); }, refill);
        rowpar_gather(ex, RS_D);
      }
      stamp(6);
      if (!st_grid_sync(a, gen)) { give_up(4); return; }
      stamp(7);

      // ================================================================ P5: norm -> silu(W1 x) * (W3 x)
      stage_norm([&](int m) -> const __half* { return a.h + (size_t)m * dim; }, L->ffn_norm);
      st_project<RS_G, NI_D, 2, MT>(hidden, KC_D, xs, M, ring, full, rg, seq, part, a, tid, no_pre,
                                         [&](int row, int m, float sa, float sb, __half) {
                                           a.ffn[(size_t)m * hidden + row] = jg_silu_mul(__float2half_rn(sa), __float2half_rn(sb));
                                         },
                                         refill);
      stamp(8);
      if (!st_grid_sync(a, gen)) { give_up(4); return; }
      stamp(9);

      // ================================================================ P6: h += W2 ffn
      stage_copy(a.ffn, hidden);
      {
        const uint32_t ex = peer_base + (uint32_t)step * ex_per_step + 2u * (uint32_t)l + 1u;
        st_project<RS_H, NI_H, 1, MT>(dim, KC_H, xs, M, ring, full, rg, seq, part, a, tid, residual,
                                      [&](int row, int m, float s, float, __half prev) { rowpar_epi(ex, row, m, s, prev); }, refill);
        rowpar_gather(ex, RS_H);
      }
      stamp(10);
      if (!st_grid_sync(a, gen)) { give_up(4); return; }
      stamp(11);
    }

    // ================================================================== final norm -> logits, (value, lowest index) key
    stage_norm([&](int m) -> const __half* { return a.h + (size_t)m * dim; }, a.out_norm);
    {
      unsigned long long best = 0ull;
      st_project<RS_D, NI_D, 1, MT>(a.vocab, KC_D, xs, M, ring, full, rg, seq, part, a, tid, no_pre,
                                         [&](int row, int m, float s, float, __half) {
                                           const __half v = __float2half_rn(s);
                                           a.logits[(size_t)m * a.vocab + row] = v;
                                           const unsigned long long k = argmax_key(v, (uint32_t)(row + a.vocab_offset));
                                           best = k > best ? k : best;
                                         },
                                         refill);
      // lane 0 of warp o finished output o = r * MT + m of every pass
      if (lane == 0 && warp < RS_D * MT && (warp % MT) < M && best != 0ull) atomicMax(a.key + (warp % MT), best);
    }
    stamp(12);
    if (!st_grid_sync(a, gen)) { give_up(4); return; }
    stamp(13);
    // every CTA reads the pick (the next step's embedding row); CTA 0 publishes it.  Under tensor parallelism every rank
    // holds the best key of its share of the vocabulary: CTA 0 sends it to all ranks as a pair of entries, and every CTA
    // of every rank takes the largest of the ranks' keys (largest value, lowest index among equals)
    if (world > 1) {
      const uint32_t ex = peer_base + (uint32_t)step * ex_per_step + 2u * (uint32_t)a.n_layers;
      constexpr size_t KEY_AT = PEER_LL_VALUES / 2;  // entries [KEY_AT, KEY_AT + 2 M): beyond any [M][dim] sum
      if (tid < M) {
        if (bid == 0) {
          const unsigned long long k = __ldcg(a.key + tid);
          for (int p = 0; p < world; p++)
            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(peer_ll(a.peer.buf[p], (int)(ex & 1u), a.peer.rank) + KEY_AT + 2 * tid),
                         "r"((uint32_t)(k & 0xFFFFFFFFull)), "r"(ex), "r"((uint32_t)(k >> 32)) : "memory");
        }
        unsigned long long best = 0ull;
        bool ok = true;
        for (int rk = 0; rk < world && ok; rk++) {
          float lo = 0.f, hi = 0.f;
          ok = peer_ll_load2(peer_ll(a.peer.buf[a.peer.rank], (int)(ex & 1u), rk) + KEY_AT + 2 * tid, ex, a.peer.timeout_ns, &lo, &hi);
          const unsigned long long k = ((unsigned long long)__float_as_uint(hi) << 32) | (unsigned long long)__float_as_uint(lo);
          best = k > best ? k : best;
        }
        if (!ok) atomicCAS(a.peer.err, 0, 1);
        s_key[tid] = best;
      }
      __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
      if (m < M) {
        const unsigned long long k = world > 1 ? s_key[m] : __ldcg(a.key + m);
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
struct jg_comm;
int jg_peer_fill_args_n(jg_comm* comm, PeerArgs* a, uint32_t count);  // comm.cu: `count` consecutive exchange numbers

struct jg_step {
  jg_dev* dev;
  jg_kvcache* kv;
  jg_comm* comm;  // tensor parallelism: the rank's communicator (peer buffers open); null on one GPU
  StepArgs args;  // everything but the per-call buffers
  StepLayer* d_layers;
  int variant[2];  // index into the instantiation table: 1-row kernel, 2-row kernel
  int grid;
  int max_rows;
  size_t smem[2];      // dynamic shared memory of the 1-row and the 2-row kernel
  int nslot[2], ring_offset[2], slot_bytes[2];
  int max_slices;
  uint64_t steps_run, launches_run;
};

typedef void (*StepKernel)(const StepArgs);
struct StepVariant { int mt, hd, nrep, rs_d, rs_g, rs_h, ni_d, ni_h; StepKernel kern; };
#define ST_VARIANT(MT, HD, NREP, RSD, RSG, RSH, NID, NIH) {MT, HD, NREP, RSD, RSG, RSH, NID, NIH, jg_step_kernel<MT, HD, NREP, RSD, RSG, RSH, NID, NIH>}
// Per model shape: the 1-row and the 2-row kernel, each with 64 KB and with 32 KB passes.
static const StepVariant g_step_variants[] = {
    // Llama-3.1-8B: dim 4096, hidden 14336
    ST_VARIANT(1, 128, 4, 8, 4, 2, 1, 4), ST_VARIANT(1, 128, 4, 4, 2, 1, 1, 4), ST_VARIANT(2, 128, 4, 4, 2, 1, 1, 4),
    ST_VARIANT(2, 128, 4, 8, 4, 2, 1, 4),
    // the same under tensor parallelism: a rank's share of the hidden width is 7168 (2 ranks), 3584 (4) or 1792 (8) columns
    ST_VARIANT(1, 128, 4, 8, 4, 4, 1, 2), ST_VARIANT(2, 128, 4, 8, 4, 4, 1, 2),
    ST_VARIANT(1, 128, 4, 8, 4, 8, 1, 1), ST_VARIANT(2, 128, 4, 8, 4, 8, 1, 1),
    // ... with 32 KB passes (more passes per CTA when a rank's matrices are small)
    ST_VARIANT(1, 128, 4, 4, 2, 2, 1, 2), ST_VARIANT(2, 128, 4, 4, 2, 2, 1, 2),
    ST_VARIANT(1, 128, 4, 4, 2, 4, 1, 1), ST_VARIANT(2, 128, 4, 4, 2, 4, 1, 1),
    ST_VARIANT(1, 128, 4, 4, 2, 8, 1, 1), ST_VARIANT(2, 128, 4, 4, 2, 8, 1, 1),
    // Llama-3.2-1B: dim 2048, hidden 8192
    ST_VARIANT(1, 64, 4, 8, 4, 4, 1, 2), ST_VARIANT(1, 64, 4, 8, 4, 2, 1, 2), ST_VARIANT(2, 64, 4, 8, 4, 2, 1, 2),
    ST_VARIANT(2, 64, 4, 8, 4, 4, 1, 2),
    // Llama-3.2-3B: dim 3072, hidden 8192
    ST_VARIANT(1, 128, 3, 8, 4, 4, 1, 2), ST_VARIANT(1, 128, 3, 5, 2, 2, 1, 2), ST_VARIANT(2, 128, 3, 5, 2, 2, 1, 2),
    ST_VARIANT(2, 128, 3, 8, 4, 4, 1, 2),
};

static int ni_for(int K) { return (K / 8 + ST_THREADS - 1) / ST_THREADS; }  // 16-byte chunks per thread and row
static int rs_for(int slot_bytes, int K, int matrices, int cap) {            // whole rows of `matrices` matrices per slot
  const int r = slot_bytes / (matrices * K * 2);
  return r < cap ? r : cap;
}
static int find_variant(int mt, int hd, int nrep, int dim, int hidden, int slot_bytes) {
  const int ni_d = ni_for(dim), ni_h = ni_for(hidden);
  const int cap = ST_WARPS / mt;  // one output per finishing warp
  const int rs_d = rs_for(slot_bytes, dim, 1, cap < 8 ? cap : 8), rs_g = rs_for(slot_bytes, dim, 2, 4), rs_h = rs_for(slot_bytes, hidden, 1, cap < 8 ? cap : 8);
  const int nv = (int)(sizeof(g_step_variants) / sizeof(g_step_variants[0]));
  for (int i = 0; i < nv; i++) {
    const StepVariant& v = g_step_variants[i];
    if (v.mt == mt && v.hd == hd && v.nrep == nrep && v.ni_d == ni_d && v.ni_h == ni_h && v.rs_d == rs_d && v.rs_g == rs_g && v.rs_h == rs_h) return i;
  }
  return -1;
}

static void step_destroy_now(void* p) {
  jg_step* s = (jg_step*)p;
  if (s->d_layers) cudaFree(s->d_layers);
  if (s->args.att_ml) cudaFree(s->args.att_ml);
  if (s->args.att_o) cudaFree(s->args.att_o);
  if (s->args.tickets) cudaFree(s->args.tickets);
  if (s->args.bar) cudaFree(s->args.bar);
  if (s->args.key) cudaFree(s->args.key);
  if (s->args.prof) {
    unsigned long long t[32];
    if (cudaMemcpy(t, s->args.prof, sizeof(t), cudaMemcpyDeviceToHost) == cudaSuccess && t[30] > 0) {
      s->steps_run = t[30];
      s->launches_run = t[14];
      static const char* names[14] = {"norm+qkv", "barrier", "scores", "barrier", "p.v+fold", "barrier", "wo", "barrier", "norm+gate/up",
                                      "barrier", "down", "barrier", "norm+logits", "barrier"};
      fprintf(stderr, "[jg_step] mean microseconds per step over %llu steps (CTA 0 | last CTA):\n", (unsigned long long)s->steps_run);
      for (int i = 0; i < 14; i++)
        fprintf(stderr, "[jg_step]   %-13s %9.1f | %9.1f\n", names[i], t[i] / 1e3 / (double)s->steps_run, t[16 + i] / 1e3 / (double)s->steps_run);
      if (s->args.bar_probe > 0)
        fprintf(stderr, "[jg_step]   %d back-to-back barriers per launch: %.2f us each\n", s->args.bar_probe,
                t[15] / 1e3 / (double)s->launches_run / s->args.bar_probe);
    }
    cudaFree(s->args.prof);
  }
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
  const int max_rows = 2;
  const int grid = dev->sm_count;
  JG_REQUIRE(grid >= max_rows * k.n_kv_heads, "step_create: fewer SMs than (row, kv head) pairs");
  // context slices per (row, kv head): as many as the CTAs allow (at most 32); one slice's scores must fit
  const int slices_min = grid / (max_rows * k.n_kv_heads) < 32 ? grid / (max_rows * k.n_kv_heads) : 32;
  const int chunk_cap = ((kv->max_ctx + slices_min - 1) / slices_min + 31) & ~31;
  const size_t att_bytes = ((size_t)nrep * chunk_cap + (size_t)(ST_WARPS / 2) * nrep * k.head_dim) * sizeof(float);
  size_t smem[2];
  int nslot[2], ring_offset[2], slot_bytes[2], variant[2];
  const char* ke = getenv("JG_STEP_SLOT_KB");
  for (int mt = 1; mt <= 2; mt++) {
    const size_t x_bytes = (size_t)mt * (d.dim > d.hidden_dim ? d.dim : d.hidden_dim) * sizeof(__half);
    const size_t head = ((att_bytes > x_bytes ? att_bytes : x_bytes) + 127) & ~(size_t)127;
    const long long room = (long long)dev->prop.sharedMemPerBlockOptin - 4096 - (long long)head;  // 4 KB: the kernel's static arrays
    // 64 KB passes (half the barriers and epilogues per byte of 32 KB ones) where at least two of them fit: three beside
    // one activation row, two beside two rows (8B shapes, two rows: 516 tok/s against 491 with five 32 KB passes)
    int sb = room >= 2 * 65536 ? 65536 : 32768;
    if (ke && atoi(ke) == 32) sb = 32768;
    int ns = (int)(room / sb);
    if (ns > ST_MAX_SLOTS) ns = ST_MAX_SLOTS;
    const char* se = getenv("JG_STEP_SLOTS");
    if (se && atoi(se) >= 2 && atoi(se) < ns) ns = atoi(se);
    const int q_dim = k.n_heads * k.head_dim;  // Wo's columns: all heads on one GPU, a rank's share under tensor parallelism
    const bool heads_ok = d.comm != 0 ? (q_dim <= d.dim && q_dim % 8 == 0) : q_dim == d.dim;
    const int vi = (heads_ok && nrep <= 4) ? find_variant(mt, k.head_dim, nrep, d.dim, d.hidden_dim, sb) : -1;
    if (ns < 2 || vi < 0) {
      jg_set_error("step_create: no single-kernel step for dim %d, hidden %d, head_dim %d, %d query heads per kv head (%d slots of %d bytes)",
                   d.dim, d.hidden_dim, k.head_dim, nrep, ns, sb);
      return JG_ENOTSUP;
    }
    nslot[mt - 1] = ns; ring_offset[mt - 1] = (int)head; slot_bytes[mt - 1] = sb; variant[mt - 1] = vi;
    smem[mt - 1] = head + (size_t)ns * sb;
  }
  int coop = 0;
  JG_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev->ordinal));
  if (!coop) { jg_set_error("step_create: the device does not support cooperative launches"); return JG_ENOTSUP; }
  for (int i = 0; i < 2; i++) {
    JG_CUDA(cudaFuncSetAttribute(g_step_variants[variant[i]].kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem[i]));
    int per_sm = 0;
    JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, g_step_variants[variant[i]].kern, ST_THREADS, smem[i]));
    if (per_sm < 1) { jg_set_error("step_create: the step kernel does not fit an SM"); return JG_ENOTSUP; }
  }
  jg_step* s = new jg_step();
  memset(s, 0, sizeof(*s));
  s->dev = dev; s->kv = kv; s->grid = grid; s->comm = (jg_comm*)(uintptr_t)d.comm; s->max_rows = max_rows; s->max_slices = 32;
  if (getenv("JG_STEP_SLICES") != nullptr && atoi(getenv("JG_STEP_SLICES")) >= slices_min) s->max_slices = atoi(getenv("JG_STEP_SLICES"));
  s->args.slice_len = (getenv("JG_STEP_SLICE_LEN") != nullptr && atoi(getenv("JG_STEP_SLICE_LEN")) > 0) ? atoi(getenv("JG_STEP_SLICE_LEN")) : 48;
  for (int i = 0; i < 2; i++) {
    s->smem[i] = smem[i]; s->nslot[i] = nslot[i]; s->ring_offset[i] = ring_offset[i]; s->slot_bytes[i] = slot_bytes[i]; s->variant[i] = variant[i];
  }
  StepArgs& a = s->args;
  a.tok_emb = (const __half*)d.tok_embeddings; a.out_norm = (const __half*)d.out_norm; a.out_w = (const __half*)d.output;
  a.table = (const __half*)d.freqs_cis; a.table_rows = d.freqs_rows;
  a.k_pool = kv->k_pool; a.v_pool = kv->v_pool; a.block_table = kv->block_table; a.layer_elems = kv->layer_elems;
  a.n_layers = d.n_layers; a.dim = d.dim; a.hidden = d.hidden_dim; a.H = k.n_heads; a.G = k.n_kv_heads; a.vocab = d.vocab_size;
  a.q_dim = k.n_heads * k.head_dim; a.embed_rows = d.embed_rows > 0 ? d.embed_rows : d.vocab_size; a.vocab_offset = d.vocab_offset;
  a.page = k.page_size; a.page_shift = ilog2(k.page_size); a.max_pages_per_seq = k.max_pages_per_seq; a.max_ctx = kv->max_ctx;
  a.chunk_cap = chunk_cap;
  a.eps = d.norm_eps; a.scale = 1.0f / sqrtf((float)k.head_dim); a.recip_dim = 1.0f / (float)d.dim;
  a.bar_probe = (getenv("JG_STEP_PROF") != nullptr && atoi(getenv("JG_STEP_PROF")) == 2) ? 64 : 0;
  const char* te = getenv("JG_STEP_TIMEOUT_MS");
  a.timeout_ns = (unsigned long long)(te ? atoll(te) : 2000) * 1000000ull;
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
  if (e == cudaSuccess && getenv("JG_STEP_PROF") != nullptr && atoi(getenv("JG_STEP_PROF")) != 0) {
    e = cudaMalloc(&a.prof, 32 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemsetAsync(a.prof, 0, 32 * sizeof(unsigned long long), dev->stream);
  }
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
  if (s->comm != nullptr) {  // 2 exchanges per layer and one for the pick, per step
    int rc = jg_peer_fill_args_n(s->comm, &a.peer, (uint32_t)n_steps * (uint32_t)(2 * a.n_layers + 1));
    if (rc) return rc;
    a.peer_ord0 = a.peer.ord;
    JG_REQUIRE((size_t)B * a.dim <= PEER_LL_VALUES / 2, "step_run: %d rows of %d values exceed the exchange entries", B, a.dim);
  }
  int sl = s->grid / (B * a.G);
  if (sl > s->max_slices) sl = s->max_slices;
  a.slices = sl;
  JG_REQUIRE((long long)sl * a.chunk_cap >= a.max_ctx, "step_run: context slices do not cover the cache");
  const int vi = B > 1 ? 1 : 0;
  const StepVariant& v = g_step_variants[s->variant[vi]];
  a.nslot = s->nslot[vi];
  a.slot_bytes = s->slot_bytes[vi];
  a.ring_offset = s->ring_offset[vi];
  // the arrival count starts at zero whatever an earlier launch that ran out of time left behind
  JG_CUDA(cudaMemsetAsync(a.bar, 0, sizeof(unsigned int), dev->stream));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(s->grid);
  cfg.blockDim = dim3(ST_THREADS);
  cfg.dynamicSmemBytes = s->smem[vi];
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, v.kern, (const StepArgs)a);
  if (e != cudaSuccess) return jg_cuda_fail(e, "step", __FILE__, __LINE__);
  s->steps_run += (uint64_t)n_steps;
  s->launches_run++;
  dev->tc_pending = true;  // the error word is looked at after the next synchronisation
  return jg_after_launch(dev, "step");
}
