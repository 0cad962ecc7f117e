// Weight-streaming matrix-vector kernels for decode (M = batch rows <= 8): y[m][n] = sum_k x[m][k] * W[n][k].
//
// The weight matrix is read exactly once per launch with 128-bit streaming loads; the activation rows live in
// shared memory.  Each CTA owns a contiguous run of row groups ("units": RW rows of one matrix, or one row of each of
// the two SwiGLU matrices).  The run is split in two parts:
//   * bulk: floor(n/8) units per warp, each warp on its own rows with RW x U independent 16-byte loads per lane in
//     flight and no synchronisation with the other warps;
//   * remainder (n mod 8 units): all eight warps work on the same rows, each on an interleaved eighth of K, and the
//     partial sums meet in shared memory.  This keeps the CTAs of a launch within one unit of each other even when
//     a matrix has only a few rows per SM (the 4096-row projections of an 8B model give 3.5 units per CTA).
// Before the kernel waits for its predecessor (programmatic dependent launch) each warp asks for the head of its
// span to be brought into L2 with a bulk prefetch: weights do not depend on the previous kernel, so they can travel
// while it drains and while the activations are staged.  Products of fp16 operands are exact in fp32 and are
// accumulated in fp32 (Tensor.dot with sum_acc_dtype: jsgrad/tensor.ts:2593-2605, jsgrad/dtype.ts:243-248); only the
// summation order differs from a sequential loop.
//
// Fused around the reduction, all from the Llama block (jsgrad/models/llama.ts:108-127,210):
//   prologue  NORM      x <- RMSNorm(x) * g            (jsgrad/nn/index.ts:586-588)
//   epilogue  RESIDUAL  y <- residual + half(acc)       (x.add(...), fp16 add)
//             SWIGLU    y <- silu(half(acc_gate)) * half(acc_up)
//             LOGITS    y <- half(acc) and (value, lowest index) folded into a 64-bit max key per row
//             PARTIAL   y32 <- acc (fp32): one rank's share of a row-parallel projection, reduced by a later call
//             PEER      y <- residual + half(sum over ranks of acc): the same share, all-reduced inside this kernel
//                       over NVLink peer memory — CTA c of every rank owns the same output rows, so it stores its
//                       partial sums, each paired with the exchange number (flag-in-data, peer.cuh), into the peers'
//                       buffers, waits (bounded) for the peers' entries of its own rows and finishes them itself; no
//                       grid-wide step and no second launch
//             PUSH      the first half of that exchange only: the entries go to every rank's buffer (this rank's
//                       included) and the kernel ends without waiting for anybody
//   prologue  GATHER    the second half, in the kernel that consumes the sum (the next norm + projection of the block):
//                       x <- h_in + half(sum over ranks of the pushed entries), then NORM on it.  The NVLink crossing
//                       of the entries thus overlaps the producer's tail, this kernel's launch and its weight
//                       prefetch instead of stalling the producer.  The CTAs of a thread-block cluster split the
//                       reduction and hand each other their slices through distributed shared memory, so each CTA
//                       reads only 1/cluster of the entries; the first cluster also writes the new residual stream
#include "common.cuh"
#include "peer.cuh"
#include "transcendental.cuh"

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_LOGITS = 3, EPI_PARTIAL = 4, EPI_PEER = 5, EPI_PUSH = 6 };

struct GemvArgs {
  const __half* x;       // [M][K]
  const __half* norm_w;  // [K] (NORM only)
  const void* w0;        // [N][K] fp16 or int8
  const void* w1;        // second matrix (SWIGLU: up projection)
  const __half* s0;      // [N] int8 scales
  const __half* s1;
  __half* y;             // [M][N]
  const __half* residual;
  unsigned long long* key;  // [M] (LOGITS)
  float* y32;               // [M][N] unrounded fp32 sums (PARTIAL: one rank's share of a row-parallel projection)
  int row_offset;           // LOGITS: vocabulary index of weight row 0 (vocabulary-sharded output layer)
  float eps, recip_k;
  int M, N, K;
  PeerArgs peer;            // PEER / PUSH / GATHER: exchange buffers of the ranks, exchange counter, error word
  const __half* h_in;       // GATHER: residual stream before the exchanged sum is added ([M][K])
  __half* h_out;            // GATHER: residual stream after it (a different buffer: other clusters still read h_in)
};

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

// int8 x16 (one uint4) -> sixteen fp32 values of half(q) * s, the fp16 product rounded once (Int8Linear:
// jsgrad/models/llama3.ts:35).  Bytes are turned into halves exactly through the 0x6400 (1024.0) exponent trick.
__device__ __forceinline__ void dequant16(const uint4& raw, __half2 s2, float (&w)[16]) {
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);  // 1024 + 128
#pragma unroll
  for (int i = 0; i < 4; i++) {
    uint32_t v = words[i] ^ 0x80808080u;                  // signed -> offset-binary
    uint32_t lo = __byte_perm(v, 0x64646464u, 0x4140);    // bytes 0,1 -> halves 0x64b0, 0x64b1
    uint32_t hi = __byte_perm(v, 0x64646464u, 0x4342);    // bytes 2,3
    __half2 a = __hsub2(*reinterpret_cast<__half2*>(&lo), bias);  // exact: integers below 2048
    __half2 b = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
    float2 fa = __half22float2(__hmul2_rn(a, s2));
    float2 fb = __half22float2(__hmul2_rn(b, s2));
    w[i * 4 + 0] = fa.x; w[i * 4 + 1] = fa.y; w[i * 4 + 2] = fb.x; w[i * 4 + 3] = fb.y;
  }
}

// Ask for `bytes` (multiple of 16) starting at `p` (16-byte aligned) to be brought into L2; returns at once.
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

constexpr uint32_t GEMV_PREFETCH_BYTES = 4096;  // per weight row and warp, ahead of the dependency wait

// Rank of this CTA in its cluster / size of the cluster (1 when the launch carries no cluster dimension).
__device__ __forceinline__ uint32_t cluster_cta_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_cta_count() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void st_cluster_u32(uint32_t local_addr, uint32_t cta, uint32_t v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(v) : "memory");
}

template <int MT, bool W8, int EPI, bool NORM, int RW, int U, bool GATHER>
__global__ void __launch_bounds__(GEMV_THREADS, 2) jg_matvec_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);  // [MT][K]
  constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
  constexpr int NACC = NW * RW;                 // weight rows of one unit
  constexpr int CH = W8 ? 16 : 8;               // weights per 16-byte load
  constexpr int GU = (8 / MT) > 0 ? (8 / MT) : 1;  // units per cooperative pass (bounds the accumulators)
  __shared__ float part[GEMV_WARPS][GU * NACC * MT];
  __shared__ float red[GEMV_WARPS];
  __shared__ float s_rs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.K, N = a.N;
  pdl_launch();

  // ---- this CTA's contiguous run of units: [u0, u1) = bulk (nb units per warp) + remainder (< 8 units)
  const int n_units = (N + RW - 1) / RW;
  const int u0 = (int)((long long)blockIdx.x * n_units / gridDim.x);
  const int u1 = (int)((long long)(blockIdx.x + 1) * n_units / gridDim.x);
  const int nb = (u1 - u0) / GEMV_WARPS;
  const int rem0 = u0 + nb * GEMV_WARPS;  // first unit of the remainder
  const int KC = K / CH;                  // 16-byte chunks per weight row
  const size_t row_bytes = W8 ? (size_t)K : (size_t)K * 2;
  const unsigned char* wbase[NW];
  wbase[0] = reinterpret_cast<const unsigned char*>(a.w0);
  if (NW == 2) wbase[NW - 1] = reinterpret_cast<const unsigned char*>(a.w1);

  // ---- L2 prefetch of the head of this warp's first rows (bulk) or of its K-slice of the shared rows (remainder)
  if (lane < NACC) {
    const int w = lane / RW, r = lane % RW;
    if (nb > 0) {
      const int row = min((u0 + warp * nb) * RW + r, N - 1);
      const uint32_t bytes = (uint32_t)min((size_t)GEMV_PREFETCH_BYTES, row_bytes);
      l2_prefetch_bulk(wbase[w] + (size_t)row * row_bytes, bytes & ~15u);
    } else if (rem0 < u1) {
      const int row = min(rem0 * RW + r, N - 1);
      const size_t off = (size_t)warp * 512;  // this warp's first 512-byte piece of the row
      if (off + 512 <= row_bytes) l2_prefetch_bulk(wbase[w] + (size_t)row * row_bytes + off, 512);
    }
  }

  // PEER / PUSH / GATHER: the exchange's number (base + ordinal; the base word only changes between runs of launches,
  // never while one is in flight, so it is read ahead of the dependency wait) and the buffer parity it selects
  uint32_t peer_epoch = 0;
  int peer_parity = 0;
  if (EPI == EPI_PEER || EPI == EPI_PUSH || GATHER) {
    peer_epoch = a.peer.epoch[0] + a.peer.ord;
    peer_parity = (int)(peer_epoch & 1u);
  }

  // ---- everything below reads what the previous kernel wrote
  pdl_wait();
  // PEER: the partial sums land in this rank's own slot first
  float* peer_mine = nullptr;
  if (EPI == EPI_PEER || EPI == EPI_PUSH) peer_mine = peer_slot(a.peer.buf[a.peer.rank], peer_parity, a.peer.rank);

  if (GATHER) {
    // ---- finish the exchange the preceding kernel of every rank started: h_out = h_in + half(sum over ranks), in
    //      rank order so that all ranks hold identical bits.  That kernel has completed on this rank (dependency wait
    //      above) and carried the same exchange number; the peers' entries may still be in flight.
    //      Each CTA of the cluster reduces its slice (pairs of values) and writes the fp16 results into the
    //      activation rows of every CTA of the cluster.
    const uint32_t ex = peer_epoch;
    const int par = peer_parity;
    const uint32_t cr = cluster_cta_rank(), cs = cluster_cta_count();
    const int pairs = a.M * K / 2;
    const int per = (pairs + (int)cs - 1) / (int)cs;
    const int p_lo = (int)cr * per, p_hi = min(pairs, p_lo + per);
    const bool writer = (blockIdx.x < cs);  // the first cluster stores the new residual stream
    bool ok = true;
    for (int pi = p_lo + tid; pi < p_hi; pi += GEMV_THREADS) {
      float s0 = 0.f, s1 = 0.f;
      for (int r = 0; r < a.peer.world && ok; r++) {
        float v0 = 0.f, v1 = 0.f;
        const uint2* e = peer_ll(a.peer.buf[a.peer.rank], par, r) + 2 * (size_t)pi;
        ok = peer_ll_load2(e, ex, a.peer.timeout_ns, &v0, &v1);
        s0 = __fadd_rn(s0, v0);
        s1 = __fadd_rn(s1, v1);
      }
      const __half2 old = *reinterpret_cast<const __half2*>(a.h_in + 2 * (size_t)pi);
      __half2 nw;
      nw.x = hadd1(old.x, __float2half_rn(s0));
      nw.y = hadd1(old.y, __float2half_rn(s1));
      const uint32_t bits = *reinterpret_cast<const uint32_t*>(&nw);
      if (writer) *reinterpret_cast<uint32_t*>(a.h_out + 2 * (size_t)pi) = bits;
      const uint32_t local = (uint32_t)__cvta_generic_to_shared(xs + 2 * (size_t)pi);
      for (uint32_t c = 0; c < cs; c++) st_cluster_u32(local, c, bits);
    }
    if (!ok) atomicCAS(a.peer.err, 0, 1);  // a peer never arrived: the step's results are void, nobody is waited for
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }

  // ---- prologue: activation rows -> shared memory (normalised when NORM); rows beyond M are zero
  for (int m = 0; m < MT; m++) {
    __half* xm = xs + (size_t)m * K;
    if (m >= a.M) {
      for (int c = tid; c < K / 8; c += GEMV_THREADS) reinterpret_cast<uint4*>(xm)[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const __half* xg = GATHER ? xm : a.x + (size_t)m * K;  // GATHER: the rows are in place already
    if (NORM) {
      float ss = 0.f;
      for (int c = tid; c < K / 8; c += GEMV_THREADS) {
        float v[8];
        unpack8(ld_128(xg + (size_t)c * 8), v);
#pragma unroll
        for (int k = 0; k < 8; k++) ss = fmaf(v[k], v[k], ss);
      }
      ss = warp_sum(ss);
      __syncthreads();  // red / s_rs reuse across rows
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      if (tid == 0) {
        float t = 0.f;
        for (int i = 0; i < GEMV_WARPS; i++) t += red[i];
        s_rs = sqrtf(__fdiv_rn(1.0f, __fadd_rn(__fmul_rn(t, a.recip_k), a.eps)));
      }
      __syncthreads();
      const float rs = s_rs;
      for (int c = tid; c < K / 8; c += GEMV_THREADS) {
        float v[8];
        unpack8(ld_128(xg + (size_t)c * 8), v);
        uint4 gv = ld_128(a.norm_w + (size_t)c * 8);
        const __half* gh = reinterpret_cast<const __half*>(&gv);
        __align__(16) __half o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = hmul1(__float2half_rn(__fmul_rn(v[k], rs)), gh[k]);
        reinterpret_cast<uint4*>(xm)[c] = *reinterpret_cast<uint4*>(o);
      }
    } else if (!GATHER) {
      for (int c = tid; c < K / 8; c += GEMV_THREADS) reinterpret_cast<uint4*>(xm)[c] = ld_128(xg + (size_t)c * 8);
    }
  }
  __syncthreads();

  unsigned long long best = 0ull;  // LOGITS: running (value, index) key of the outputs this thread stores

  // One 16-byte chunk `c` of weight row data `wv` against the activations: acc[m] += sum_k w[k] * x[m][k].
  auto fma_chunk = [&](float (&acc)[MT], const uint4& wv, int c, __half2 sc) {
    if (!W8) {
#pragma unroll
      for (int m = 0; m < MT; m++) {
        float xf[8];
        unpack8(*reinterpret_cast<const uint4*>(xs + (size_t)m * K + (size_t)c * 8), xf);
        acc[m] = dot8_acc(acc[m], wv, xf);
      }
    } else {
      float wf[16];
      dequant16(wv, sc, wf);
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * K + (size_t)c * 16);
        float lo[8], hi[8];
        unpack8(xp[0], lo);
        unpack8(xp[1], hi);
#pragma unroll
        for (int k = 0; k < 8; k++) acc[m] = fmaf(wf[k], lo[k], acc[m]);
#pragma unroll
        for (int k = 0; k < 8; k++) acc[m] = fmaf(wf[8 + k], hi[k], acc[m]);
      }
    }
  };
  // Final value of output (row, m) from the reduced sums of its NW matrices.
  auto finish = [&](int row, int m, float s_a, float s_b) {
    const size_t o = (size_t)m * N + (size_t)row;
    if (EPI == EPI_PARTIAL) { a.y32[o] = s_a; return; }
    if (EPI == EPI_PEER) {  // own slot (read back in the tail) and, right away, the peers' buffers: the NVLink crossing
      peer_mine[o] = s_a;   // overlaps whatever this CTA still has to compute
      for (int p = 0; p < a.peer.world; p++)
        if (p != a.peer.rank) peer_ll_store(peer_ll(a.peer.buf[p], peer_parity, a.peer.rank) + o, s_a, peer_epoch);
      return;
    }
    if (EPI == EPI_PUSH) {  // flag-in-data entry for every rank, this one included; nothing is awaited here
      for (int p = 0; p < a.peer.world; p++) peer_ll_store(peer_ll(a.peer.buf[p], peer_parity, a.peer.rank) + o, s_a, peer_epoch);
      return;
    }
    __half v = __float2half_rn(s_a);
    if (EPI == EPI_RESIDUAL) v = hadd1(a.residual[o], v);
    if (EPI == EPI_SWIGLU) v = jg_silu_mul(v, __float2half_rn(s_b));
    a.y[o] = v;
    if (EPI == EPI_LOGITS) {
      const unsigned long long k = argmax_key(v, (uint32_t)(row + a.row_offset));
      best = k > best ? k : best;
    }
  };

  // ---- bulk: warp-private units
  for (int unit = u0 + warp * nb; unit < u0 + (warp + 1) * nb; unit++) {
    float acc[NACC][MT];
    const unsigned char* wrow[NACC];
    __half2 sc[NACC];
#pragma unroll
    for (int j = 0; j < NACC; j++) {
#pragma unroll
      for (int m = 0; m < MT; m++) acc[j][m] = 0.f;
      const int row = min(unit * RW + (j % RW), N - 1);  // clamp: a duplicate row is computed but never stored
      wrow[j] = wbase[j / RW] + (size_t)row * row_bytes;
      sc[j] = W8 ? __half2half2((j / RW == 0 ? a.s0 : a.s1)[row]) : __half2();
    }
    for (int c0 = lane; c0 < KC; c0 += 32 * U) {
      uint4 wv[NACC][U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int c = c0 + 32 * u;
#pragma unroll
        for (int j = 0; j < NACC; j++) wv[j][u] = (c < KC) ? ld_stream_128(wrow[j] + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int c = c0 + 32 * u;
        if (c < KC) {
#pragma unroll
          for (int j = 0; j < NACC; j++) fma_chunk(acc[j], wv[j][u], c, sc[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NACC; j++)
#pragma unroll
      for (int m = 0; m < MT; m++) acc[j][m] = warp_sum(acc[j][m]);
#pragma unroll
    for (int r = 0; r < RW; r++)
#pragma unroll
      for (int m = 0; m < MT; m++)
        if (lane == ((r * MT + m) & 31) && unit * RW + r < N && m < a.M) finish(unit * RW + r, m, acc[r][m], acc[(NW - 1) * RW + r][m]);
  }

  // ---- remainder: all warps on the same units, K split between the warps in 512-byte pieces
  for (int g0 = rem0; g0 < u1; g0 += GU) {
    const int gu = min(GU, u1 - g0);
    float acc[GU * NACC][MT];
#pragma unroll
    for (int j = 0; j < GU * NACC; j++)
#pragma unroll
      for (int m = 0; m < MT; m++) acc[j][m] = 0.f;
    for (int c = warp * 32 + lane; c < KC; c += GEMV_THREADS) {
      uint4 wv[GU * NACC];
#pragma unroll
      for (int j = 0; j < GU * NACC; j++) {
        const int unit = g0 + j / NACC, jj = j % NACC;
        const int row = min(unit * RW + (jj % RW), N - 1);
        wv[j] = (j / NACC < gu) ? ld_stream_128(wbase[jj / RW] + (size_t)row * row_bytes + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < GU * NACC; j++) {
        if (j / NACC < gu) {
          const int unit = g0 + j / NACC, jj = j % NACC;
          const int row = min(unit * RW + (jj % RW), N - 1);
          fma_chunk(acc[j], wv[j], c, W8 ? __half2half2((jj / RW == 0 ? a.s0 : a.s1)[row]) : __half2());
        }
      }
    }
#pragma unroll
    for (int j = 0; j < GU * NACC; j++)
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const float v = warp_sum(acc[j][m]);
        if (lane == 0) part[warp][j * MT + m] = v;
      }
    __syncthreads();
    if (tid < gu * RW * MT) {
      const int ul = tid / (RW * MT), r = (tid / MT) % RW, m = tid % MT;
      const int row = (g0 + ul) * RW + r;
      if (row < N && m < a.M) {
        float s_a = 0.f, s_b = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; w++) s_a += part[w][(ul * NACC + r) * MT + m];
        if (NW == 2) {
#pragma unroll
          for (int w = 0; w < GEMV_WARPS; w++) s_b += part[w][(ul * NACC + (NW - 1) * RW + r) * MT + m];
        }
        finish(row, m, s_a, s_b);
      }
    }
    __syncthreads();  // `part` is rewritten by the next pass
  }

  if (EPI == EPI_PEER) {
    // ---- all-reduce of this CTA's output rows [r_lo, r_hi) with CTA blockIdx.x of the other ranks, then the residual
    //      add.  Each thread carries its outputs through the whole exchange (flag-in-data entries, see peer.cuh).
    const int r_lo = u0 * RW, r_hi = min(u1 * RW, N), nr = r_hi - r_lo;
    const int rank = a.peer.rank, world = a.peer.world;
    __syncthreads();  // the partial sums written by other threads of this CTA are visible
    bool ok = true;
    for (int i = tid; i < nr * a.M; i += GEMV_THREADS) {
      const size_t o = (size_t)(i / nr) * N + r_lo + (i % nr);
      float sum = 0.f;
      for (int r = 0; r < world && ok; r++) {  // rank order on every rank: identical sums everywhere
        float v = peer_mine[o];
        if (r != rank) ok = peer_ll_load(peer_ll(a.peer.buf[rank], peer_parity, r) + o, peer_epoch, a.peer.timeout_ns, &v);
        sum = __fadd_rn(sum, v);
      }
      if (ok) a.y[o] = hadd1(a.residual[o], __float2half_rn(sum));
    }
    if (!ok) atomicCAS(a.peer.err, 0, 1);
  }

  if (EPI == EPI_LOGITS) {
    // every thread may have stored outputs of some batch row m (bulk: lane r*MT+m; remainder: tid % MT)
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const bool mine = ((lane % MT) == m) || ((tid % MT) == m);
      unsigned long long b = mine ? best : 0ull;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
        b = other > b ? other : b;
      }
      if (lane == 0 && m < a.M && b != 0ull) atomicMax(a.key + m, b);
    }
  }
}

// ------------------------------------------------------------------------------------------------ host side
template <int MT, bool W8, int EPI, bool NORM, bool GATHER = false>
static int launch_gemv(jg_dev* dev, const GemvArgs& a, const char* name) {
  // one unit = RW rows of one matrix, or one row of each SwiGLU matrix: two weight rows either way, with U chunks
  // of each in flight per lane in the warp-private part
  constexpr int RW = (EPI == EPI_SWIGLU) ? 1 : 2;
  constexpr int U = W8 ? (MT == 1 ? 4 : 2) : (MT == 1 ? 8 : (MT == 2 ? 4 : 2));
  auto kern = jg_matvec_kernel<MT, W8, EPI, NORM, RW, U, GATHER>;
  const size_t smem = (size_t)MT * a.K * sizeof(__half);
  if (smem + 2048 > (size_t)dev->prop.sharedMemPerBlockOptin) {
    jg_set_error("%s: %d activation rows of K=%d need %zu B of shared memory (limit %zu)", name, MT, a.K, smem,
                 (size_t)dev->prop.sharedMemPerBlockOptin);
    return JG_ENOTSUP;
  }
  static size_t smem_set[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // per device ordinal, per instantiation
  static int occ_for[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  static size_t occ_smem[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  static int cluster_for[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // GATHER: cluster size and how many CTAs of it fit at once
  static int cluster_ctas[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int slot = dev->ordinal & 7;
  if (smem > 48 * 1024 && smem > smem_set[slot]) {
    JG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev->prop.sharedMemPerBlockOptin - 2048));
    smem_set[slot] = dev->prop.sharedMemPerBlockOptin;
  }
  if (occ_for[slot] == 0 || occ_smem[slot] != smem) {
    int occ = 0;
    JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, GEMV_THREADS, smem));
    occ_for[slot] = occ < 1 ? 1 : (occ > 4 ? 4 : occ);
    occ_smem[slot] = smem;
    if (GATHER) {
      // the largest cluster (8, 4, 2) that still lets (nearly) as many CTAs run at once as an unclustered launch:
      // a cluster must fit inside one GPC, so big clusters can leave SMs of a GPC without a CTA
      const int want = dev->sm_count * occ_for[slot];
      int best_cs = 1, best_ctas = want;
      static int forced = -1;
      if (forced < 0) { const char* e = getenv("JG_TP_CLUSTER"); forced = e ? atoi(e) : 0; }
      for (int cs = 8; cs >= 2; cs >>= 1) {
        if (forced > 0 && cs != forced) continue;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(want / cs * cs));
        cfg.blockDim = dim3(GEMV_THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = (unsigned)cs; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); continue; }
        if (n * cs * 100 >= want * 93 || forced > 0) { best_cs = cs; best_ctas = n * cs < want ? n * cs : want / cs * cs; break; }
      }
      cluster_for[slot] = best_cs;
      cluster_ctas[slot] = best_ctas;
    }
  }
  const int n_units = (a.N + RW - 1) / RW;
  long long blocks = (long long)dev->sm_count * occ_for[slot];
  if (blocks > n_units) blocks = n_units;
  if (EPI == EPI_PEER && blocks > PEER_MAX_CTAS) blocks = PEER_MAX_CTAS;  // one flag row per CTA
  if (blocks < 1) blocks = 1;
  int cs = 1;
  if (GATHER) {
    cs = cluster_for[slot] > 0 ? cluster_for[slot] : 1;
    if (cs > 1 && blocks > cluster_ctas[slot]) blocks = cluster_ctas[slot];
    blocks = (blocks + cs - 1) / cs * cs;  // whole clusters; a CTA without units still takes part in the gather
  }
  return jg_launch_cluster(dev, name, kern, dim3((unsigned)blocks), dim3(GEMV_THREADS), smem, cs, a);
}

// gemm_small.cu: mma.sync projection for up to 64 rows (fp16 or int8 weights, activations already normalised)
int jg_gemm_small(jg_dev* dev, int epi, const void* x, const void* w0, const void* w1, const void* s0, const void* s1,
                  void* y, const void* residual, void* key, int M, int N, int K, int row_offset);

// matvec_w8.cu: int8 weights, up to 8 rows, activations resident in shared memory (optionally normalised there)
int jg_matvec_w8(jg_dev* dev, int epi, const void* x, const void* norm_w, float eps, const void* w0, const void* w1,
                 const void* s0, const void* s1, void* y, const void* residual, void* key, int M, int N, int K, int row_offset);
bool jg_matvec_w8_fits(const jg_dev* dev, int M, int K);

// gemm_tc.cu: tcgen05 / TMA projection (fp16 weights, N % 128 == 0, K % 64 == 0), any number of rows
int jg_gemm_tc(jg_dev* dev, int epi, const void* x, const void* w0, const void* w1, void* y, const void* residual, int M, int N, int K,
               const void* s0, const void* s1);
bool jg_gemm_tc_fits(int N, int K);

// Fewest rows that go to the tcgen05 kernel when the shape allows it (JG_TC_MIN_M overrides; above 64 rows it is
// the only kernel).  Measured on the 8B shapes: 3.73 against 3.94 ms per step at 4 rows, 3.85 against 4.16 at 8.
static int tc_min_rows() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("JG_TC_MIN_M");
    v = e ? atoi(e) : 3;
    if (v < 1) v = 1;
    if (v > 65) v = 65;
  }
  return v;
}

static bool w8_mma() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("JG_W8_MMA"); v = (e && atoi(e) == 0) ? 0 : 1; }
  return v != 0;
}

static bool w8_tc() {  // JG_W8_TC=0: int8 projections of more than 64 rows are refused (the caller dequantises to fp16 first)
  static int v = -1;
  if (v < 0) { const char* e = getenv("JG_W8_TC"); v = (e && atoi(e) == 0) ? 0 : 1; }
  return v != 0;
}

// int8 weights: from this many rows on the tcgen05 kernel with the conversion inside it is ahead of the mma.sync
// kernel (8B int8 decode, ms per step, mma.sync / tcgen05: 8 rows 3.79 / 4.82, 16 rows 4.30 / 4.76, 24 rows 5.34 /
// 4.87, 32 rows 5.73 / 4.96, 48 rows 10.7 / 6.65, 64 rows 11.3 / 6.84).  JG_W8_TC_MIN overrides.
static int w8_tc_min_rows() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("JG_W8_TC_MIN"); v = e ? atoi(e) : 20; if (v < 3) v = 3; }
  return v;
}

template <bool W8, int EPI, bool NORM>
static int dispatch_m(jg_dev* dev, const GemvArgs& a, const char* name) {
  if (EPI == EPI_PEER || EPI == EPI_PUSH) {  // fused with its all-reduce: matrix-vector kernels only (up to 8 rows)
    if (a.M == 1) return launch_gemv<1, W8, EPI, NORM>(dev, a, name);
    if (a.M == 2) return launch_gemv<2, W8, EPI, NORM>(dev, a, name);
    if (a.M <= 4) return launch_gemv<4, W8, EPI, NORM>(dev, a, name);
    if (a.M <= 8) return launch_gemv<8, W8, EPI, NORM>(dev, a, name);
    jg_set_error("%s: the projection fused with its all-reduce takes at most 8 rows (M=%d)", name, a.M);
    return JG_ENOTSUP;
  }
  if (!W8 && !NORM && EPI != EPI_LOGITS && (a.M > 64 || (a.M >= tc_min_rows() && jg_gemm_tc_fits(a.N, a.K))))
    return jg_gemm_tc(dev, EPI, a.x, a.w0, a.w1, EPI == EPI_PARTIAL ? (void*)a.y32 : (void*)a.y, a.residual, a.M, a.N, a.K, nullptr, nullptr);
  // int8 weights and enough rows: the tcgen05 kernel with the conversion inside it
  if (W8 && !NORM && EPI != EPI_LOGITS && a.M >= w8_tc_min_rows() && jg_gemm_tc_fits(a.N, a.K) && w8_tc())
    return jg_gemm_tc(dev, EPI, a.x, a.w0, a.w1, EPI == EPI_PARTIAL ? (void*)a.y32 : (void*)a.y, a.residual, a.M, a.N, a.K, a.s0, a.s1);
  // int8 weights, up to 8 rows: the kernel that keeps the rows in shared memory and streams the weights through the
  // tensor cores without a barrier in its k loop; it also takes the norm in its prologue
  if (W8 && a.M <= 8 && w8_mma() && jg_matvec_w8_fits(dev, a.M, a.K) && getenv("JG_W8_RESIDENT_X") == nullptr)
    return jg_matvec_w8(dev, EPI, a.x, NORM ? a.norm_w : nullptr, a.eps, a.w0, a.w1, a.s0, a.s1,
                        EPI == EPI_PARTIAL ? (void*)a.y32 : (void*)a.y, a.residual, a.key, a.M, a.N, a.K, a.row_offset);
  // int8 weights: the CUDA-core kernel spends its issue slots on dequantisation (half(q) * scale, widen, FMA: about 80
  // instructions per 16 bytes) and reaches half of the HBM rate; on the tensor cores the widening and the FMAs are
  // gone, so pre-normalised int8 projections of any row count go to the mma.sync kernel (JG_W8_MMA=0 keeps the
  // CUDA-core kernel)
  if (W8 && !NORM && a.K >= 256 && w8_mma()) return jg_gemm_small(dev, EPI, a.x, a.w0, a.w1, a.s0, a.s1, EPI == EPI_PARTIAL ? (void*)a.y32 : (void*)a.y, a.residual, a.key, a.M, a.N, a.K, a.row_offset);
  if (a.M == 1) return launch_gemv<1, W8, EPI, NORM>(dev, a, name);
  if (a.M == 2) return launch_gemv<2, W8, EPI, NORM>(dev, a, name);
  // from 3 rows on the CUDA cores cannot keep up with the weight stream: unnormalised fp16 projections go to the
  // tensor-core kernel (measured on the 8B shapes: 48 us against 69 us at 4 rows and 106 us at 8 rows)
  if (!W8 && !NORM && a.M >= 3 && a.M <= 64 && a.K >= 256) return jg_gemm_small(dev, EPI, a.x, a.w0, a.w1, a.s0, a.s1, EPI == EPI_PARTIAL ? (void*)a.y32 : (void*)a.y, a.residual, a.key, a.M, a.N, a.K, a.row_offset);
  if (a.M <= 4) return launch_gemv<4, W8, EPI, NORM>(dev, a, name);
  if (a.M <= 8) return launch_gemv<8, W8, EPI, NORM>(dev, a, name);
  if (!NORM && a.M <= 64) return jg_gemm_small(dev, EPI, a.x, a.w0, a.w1, a.s0, a.s1, EPI == EPI_PARTIAL ? (void*)a.y32 : (void*)a.y, a.residual, a.key, a.M, a.N, a.K, a.row_offset);
  if (NORM) jg_set_error("%s: with M=%d rows (> 8) normalise first (jg_rmsnorm) and pass norm_w = 0", name, a.M);
  else if (W8) jg_set_error("%s: M=%d rows (> 64) with int8 weights: split the rows into chunks of 64", name, a.M);
  else jg_set_error("%s: M=%d rows is beyond the projection kernels (max 64 per call)", name, a.M);
  return JG_ENOTSUP;
}

static int check_common(const char* name, uint64_t y, uint64_t x, uint64_t w, uint64_t scale, int M, int N, int K) {
  JG_REQUIRE(M > 0 && N > 0 && K > 0, "%s: bad shape M=%d N=%d K=%d", name, M, N, K);
  JG_REQUIRE(K % (scale ? 16 : 8) == 0, "%s: K=%d must be a multiple of %d", name, K, scale ? 16 : 8);
  JG_REQUIRE(jg_aligned(y, 2) && jg_aligned(x, 16) && jg_aligned(w, 16), "%s: null or misaligned pointer", name);
  JG_REQUIRE(scale == 0 || jg_aligned(scale, 2), "%s: misaligned scale pointer", name);
  return JG_OK;
}

JG_API int jg_linear(jg_dev* dev, uint64_t y, uint64_t x, uint64_t w, uint64_t scale, uint64_t residual, int32_t M,
                     int32_t N, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("linear", y, x, w, scale, M, N, K);
  if (rc) return rc;
  GemvArgs a = {};
  a.x = (const __half*)x; a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)y;
  a.residual = (const __half*)residual; a.M = M; a.N = N; a.K = K;
  jg_mark_fresh(dev, y, (uint64_t)M * N * 2);  // an output may be the next call's weight matrix
  if (residual) {
    JG_REQUIRE(jg_aligned(residual, 2), "linear: misaligned residual pointer");
    return scale ? dispatch_m<true, EPI_RESIDUAL, false>(dev, a, "linear") : dispatch_m<false, EPI_RESIDUAL, false>(dev, a, "linear");
  }
  return scale ? dispatch_m<true, EPI_STORE, false>(dev, a, "linear") : dispatch_m<false, EPI_STORE, false>(dev, a, "linear");
}

JG_API int jg_norm_linear(jg_dev* dev, uint64_t y, uint64_t x, uint64_t norm_w, float eps, uint64_t w, uint64_t scale,
                          int32_t M, int32_t N, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("norm_linear", y, x, w, scale, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(norm_w, 16), "norm_linear: null or misaligned norm weight");
  GemvArgs a = {};
  a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.eps = eps; a.recip_k = (float)(1.0 / (double)K);
  a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)y; a.M = M; a.N = N; a.K = K;
  jg_mark_fresh(dev, y, (uint64_t)M * N * 2);
  return scale ? dispatch_m<true, EPI_STORE, true>(dev, a, "norm_linear") : dispatch_m<false, EPI_STORE, true>(dev, a, "norm_linear");
}

JG_API int jg_norm_swiglu(jg_dev* dev, uint64_t y, uint64_t x, uint64_t norm_w, float eps, uint64_t w_gate,
                          uint64_t s_gate, uint64_t w_up, uint64_t s_up, int32_t M, int32_t N, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("norm_swiglu", y, x, w_gate, s_gate, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(w_up, 16), "norm_swiglu: null or misaligned up-projection weight");
  JG_REQUIRE((s_gate == 0) == (s_up == 0), "norm_swiglu: gate and up projections must share a weight format");
  GemvArgs a = {};
  a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.eps = eps; a.recip_k = (float)(1.0 / (double)K);
  a.w0 = (const void*)w_gate; a.w1 = (const void*)w_up; a.s0 = (const __half*)s_gate; a.s1 = (const __half*)s_up;
  a.y = (__half*)y; a.M = M; a.N = N; a.K = K;
  if (norm_w) {
    JG_REQUIRE(jg_aligned(norm_w, 16), "norm_swiglu: misaligned norm weight");
    return s_gate ? dispatch_m<true, EPI_SWIGLU, true>(dev, a, "norm_swiglu") : dispatch_m<false, EPI_SWIGLU, true>(dev, a, "norm_swiglu");
  }
  return s_gate ? dispatch_m<true, EPI_SWIGLU, false>(dev, a, "norm_swiglu") : dispatch_m<false, EPI_SWIGLU, false>(dev, a, "norm_swiglu");
}

static int logits_impl(jg_dev* dev, uint64_t logits, uint64_t key, uint64_t x, uint64_t norm_w, float eps, uint64_t w,
                       uint64_t scale, int32_t M, int32_t V, int32_t K, int32_t row_offset);

JG_API int jg_norm_logits_argmax(jg_dev* dev, uint64_t logits, uint64_t key, uint64_t x, uint64_t norm_w, float eps,
                                 uint64_t w, uint64_t scale, int32_t M, int32_t V, int32_t K) {
  return logits_impl(dev, logits, key, x, norm_w, eps, w, scale, M, V, K, 0);
}

JG_API int jg_norm_logits_argmax_shard(jg_dev* dev, uint64_t logits, uint64_t key, uint64_t x, uint64_t norm_w, float eps,
                                       uint64_t w, uint64_t scale, int32_t M, int32_t V_local, int32_t K, int32_t row_offset) {
  JG_REQUIRE(row_offset >= 0, "norm_logits_argmax_shard: negative row offset");
  return logits_impl(dev, logits, key, x, norm_w, eps, w, scale, M, V_local, K, row_offset);
}

JG_API int jg_linear_partial(jg_dev* dev, uint64_t y32, uint64_t x, uint64_t w, uint64_t scale, int32_t M, int32_t N, int32_t K) {
  JG_ENTER(dev);
  int rc = check_common("linear_partial", y32, x, w, scale, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(y32, 4), "linear_partial: misaligned output");
  GemvArgs a = {};
  a.x = (const __half*)x; a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y32 = (float*)y32; a.M = M; a.N = N; a.K = K;
  return scale ? dispatch_m<true, EPI_PARTIAL, false>(dev, a, "linear_partial") : dispatch_m<false, EPI_PARTIAL, false>(dev, a, "linear_partial");
}

static int logits_impl(jg_dev* dev, uint64_t logits, uint64_t key, uint64_t x, uint64_t norm_w, float eps, uint64_t w,
                       uint64_t scale, int32_t M, int32_t V, int32_t K, int32_t row_offset) {
  JG_ENTER(dev);
  int rc = check_common("norm_logits_argmax", logits, x, w, scale, M, V, K);
  if (rc) return rc;
  JG_REQUIRE((norm_w == 0 || jg_aligned(norm_w, 16)) && jg_aligned(key, 8), "norm_logits_argmax: null or misaligned pointer");
  GemvArgs a = {};
  a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.eps = eps; a.recip_k = (float)(1.0 / (double)K);
  a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)logits; a.key = (unsigned long long*)key;
  a.M = M; a.N = V; a.K = K; a.row_offset = row_offset;
  if (norm_w == 0) return scale ? dispatch_m<true, EPI_LOGITS, false>(dev, a, "norm_logits_argmax") : dispatch_m<false, EPI_LOGITS, false>(dev, a, "norm_logits_argmax");
  return scale ? dispatch_m<true, EPI_LOGITS, true>(dev, a, "norm_logits_argmax") : dispatch_m<false, EPI_LOGITS, true>(dev, a, "norm_logits_argmax");
}

// h <- h + half( sum over ranks of x . W^T ): a row-parallel projection (this rank holds a K-slice of W) fused with its
// all-reduce over NVLink peer memory and the residual add of TransformerBlock.call (jsgrad/models/llama.ts:125-126), one
// launch per rank, up to 8 rows.  Every rank must call it with the same shapes, in the same order relative to its other
// peer reductions.  Needs jg_comm_peer_open; M * N is limited by the exchange buffer.
jg_dev* jg_comm_device(jg_comm* comm);
JG_API int jg_linear_allreduce_residual(jg_comm* comm, uint64_t h, uint64_t x, uint64_t w, uint64_t scale, int32_t M,
                                        int32_t N, int32_t K) {
  JG_REQUIRE(comm != nullptr, "linear_allreduce_residual: null communicator");
  jg_dev* dev = jg_comm_device(comm);
  JG_ENTER(dev);
  int rc = check_common("linear_allreduce_residual", h, x, w, scale, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(M <= 8 && (size_t)M * N <= PEER_LL_VALUES, "linear_allreduce_residual: M=%d N=%d exceed 8 rows / %zu outputs",
             M, N, (size_t)PEER_LL_VALUES);
  GemvArgs a = {};
  a.x = (const __half*)x; a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)h; a.residual = (const __half*)h;
  a.M = M; a.N = N; a.K = K;
  rc = jg_peer_fill_args(comm, &a.peer);
  if (rc) return rc;
  return scale ? dispatch_m<true, EPI_PEER, false>(dev, a, "linear_allreduce_residual")
               : dispatch_m<false, EPI_PEER, false>(dev, a, "linear_allreduce_residual");
}

// ------------------------------------------------------------------------------------------------ split exchange
// The same all-reduce cut in two, so that no kernel waits for another rank while it has nothing else to do:
//   jg_tp_linear_push        a row-parallel projection whose epilogue stores this rank's fp32 partial sums, paired with
//                            the exchange number, into every rank's buffer and returns;
//   jg_tp_norm_linear /      the projection that consumes the sum (the next norm + projection of the block, or the
//   jg_tp_norm_swiglu /      output layer): its prologue adds the ranks' entries in rank order, rounds once, adds the
//   jg_tp_norm_logits_argmax residual stream h_in, leaves the new stream in h_out and normalises it.
// Every push must be followed, on every rank, by exactly one consuming call with the same M and K = the push's N before
// the next exchange of any kind.  h_in and h_out must be different buffers.
template <bool W8, int EPI>
static int dispatch_gather(jg_dev* dev, const GemvArgs& a, const char* name) {
  if (a.M == 1) return launch_gemv<1, W8, EPI, true, true>(dev, a, name);
  if (a.M == 2) return launch_gemv<2, W8, EPI, true, true>(dev, a, name);
  if (a.M <= 4) return launch_gemv<4, W8, EPI, true, true>(dev, a, name);
  if (a.M <= 8) return launch_gemv<8, W8, EPI, true, true>(dev, a, name);
  jg_set_error("%s: the projection that gathers a pushed sum takes at most 8 rows (M=%d)", name, a.M);
  return JG_ENOTSUP;
}

static int check_gather(const char* name, jg_comm* comm, uint64_t h_out, uint64_t h_in, uint64_t norm_w, int M, int K, GemvArgs* a) {
  JG_REQUIRE(jg_aligned(h_out, 4) && jg_aligned(h_in, 4) && h_out != h_in, "%s: h_in and h_out must be two distinct, 4-byte aligned buffers", name);
  JG_REQUIRE(jg_aligned(norm_w, 16), "%s: null or misaligned norm weight", name);
  JG_REQUIRE(M <= 8 && (size_t)M * K <= PEER_LL_VALUES, "%s: M=%d K=%d exceed 8 rows / %zu exchanged values", name, M, K, (size_t)PEER_LL_VALUES);
  a->h_in = (const __half*)h_in; a->h_out = (__half*)h_out; a->norm_w = (const __half*)norm_w;
  a->recip_k = (float)(1.0 / (double)K);
  return jg_peer_fill_args(comm, &a->peer, /*consume=*/true);
}

JG_API int jg_tp_linear_push(jg_comm* comm, uint64_t x, uint64_t w, uint64_t scale, int32_t M, int32_t N, int32_t K) {
  JG_REQUIRE(comm != nullptr, "tp_linear_push: null communicator");
  jg_dev* dev = jg_comm_device(comm);
  JG_ENTER(dev);
  int rc = check_common("tp_linear_push", x, x, w, scale, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(M <= 8 && (size_t)M * N <= PEER_LL_VALUES && N % 2 == 0, "tp_linear_push: M=%d N=%d exceed 8 rows / %zu outputs (N even)", M, N,
             (size_t)PEER_LL_VALUES);
  GemvArgs a = {};
  a.x = (const __half*)x; a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.M = M; a.N = N; a.K = K;
  rc = jg_peer_fill_args(comm, &a.peer);
  if (rc) return rc;
  return scale ? dispatch_m<true, EPI_PUSH, false>(dev, a, "tp_linear_push") : dispatch_m<false, EPI_PUSH, false>(dev, a, "tp_linear_push");
}

JG_API int jg_tp_norm_linear(jg_comm* comm, uint64_t y, uint64_t h_out, uint64_t h_in, uint64_t norm_w, float eps, uint64_t w,
                             uint64_t scale, int32_t M, int32_t N, int32_t K) {
  JG_REQUIRE(comm != nullptr, "tp_norm_linear: null communicator");
  jg_dev* dev = jg_comm_device(comm);
  JG_ENTER(dev);
  int rc = check_common("tp_norm_linear", y, h_in, w, scale, M, N, K);
  if (rc) return rc;
  GemvArgs a = {};
  rc = check_gather("tp_norm_linear", comm, h_out, h_in, norm_w, M, K, &a);
  if (rc) return rc;
  a.eps = eps; a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)y; a.M = M; a.N = N; a.K = K;
  jg_mark_fresh(dev, y, (uint64_t)M * N * 2);
  return scale ? dispatch_gather<true, EPI_STORE>(dev, a, "tp_norm_linear") : dispatch_gather<false, EPI_STORE>(dev, a, "tp_norm_linear");
}

JG_API int jg_tp_norm_swiglu(jg_comm* comm, uint64_t y, uint64_t h_out, uint64_t h_in, uint64_t norm_w, float eps, uint64_t w_gate,
                             uint64_t s_gate, uint64_t w_up, uint64_t s_up, int32_t M, int32_t N, int32_t K) {
  JG_REQUIRE(comm != nullptr, "tp_norm_swiglu: null communicator");
  jg_dev* dev = jg_comm_device(comm);
  JG_ENTER(dev);
  int rc = check_common("tp_norm_swiglu", y, h_in, w_gate, s_gate, M, N, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(w_up, 16), "tp_norm_swiglu: null or misaligned up-projection weight");
  JG_REQUIRE((s_gate == 0) == (s_up == 0), "tp_norm_swiglu: gate and up projections must share a weight format");
  GemvArgs a = {};
  rc = check_gather("tp_norm_swiglu", comm, h_out, h_in, norm_w, M, K, &a);
  if (rc) return rc;
  a.eps = eps; a.w0 = (const void*)w_gate; a.w1 = (const void*)w_up; a.s0 = (const __half*)s_gate; a.s1 = (const __half*)s_up;
  a.y = (__half*)y; a.M = M; a.N = N; a.K = K;
  return s_gate ? dispatch_gather<true, EPI_SWIGLU>(dev, a, "tp_norm_swiglu") : dispatch_gather<false, EPI_SWIGLU>(dev, a, "tp_norm_swiglu");
}

JG_API int jg_tp_norm_logits_argmax(jg_comm* comm, uint64_t logits, uint64_t key, uint64_t h_out, uint64_t h_in, uint64_t norm_w,
                                    float eps, uint64_t w, uint64_t scale, int32_t M, int32_t V_local, int32_t K, int32_t row_offset) {
  JG_REQUIRE(comm != nullptr, "tp_norm_logits_argmax: null communicator");
  jg_dev* dev = jg_comm_device(comm);
  JG_ENTER(dev);
  int rc = check_common("tp_norm_logits_argmax", logits, h_in, w, scale, M, V_local, K);
  if (rc) return rc;
  JG_REQUIRE(jg_aligned(key, 8) && row_offset >= 0, "tp_norm_logits_argmax: misaligned key buffer or negative row offset");
  GemvArgs a = {};
  rc = check_gather("tp_norm_logits_argmax", comm, h_out, h_in, norm_w, M, K, &a);
  if (rc) return rc;
  a.eps = eps; a.w0 = (const void*)w; a.s0 = (const __half*)scale; a.y = (__half*)logits; a.key = (unsigned long long*)key;
  a.M = M; a.N = V_local; a.K = K; a.row_offset = row_offset;
  return scale ? dispatch_gather<true, EPI_LOGITS>(dev, a, "tp_norm_logits_argmax") : dispatch_gather<false, EPI_LOGITS>(dev, a, "tp_norm_logits_argmax");
}
