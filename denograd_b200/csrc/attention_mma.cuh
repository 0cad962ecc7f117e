// Decode attention on the tensor cores: the same one-launch cluster scheme as attn_decode_fused_kernel (RoPE, cache
// write, scores, softmax statistics over distributed shared memory, p.v, cross-CTA fold; see attention.cu) with the two
// context loops restated as mma.sync.m16n8k16 products over K / V tiles staged in shared memory by cp.async:
//   scores^T [16 positions x 8 heads] = K tile [16 x hd] . q^T [hd x 8]      (heads beyond n_rep are padding)
//   out^T    [16 dims x 8 heads]     = V^T tile [16 x 16 positions] . p^T     (V^T fragments via ldmatrix.trans)
// With many rows in flight (batched decode over long contexts) the CUDA-core loops of the original kernel are bound by
// their shuffle reductions, not by the KV stream; here a warp issues 8 MMAs per 16 positions and the loads are
// asynchronous 16-byte copies.  Arithmetic: fp32 accumulation of exact fp16 products (order differs), scores scaled in
// fp32, p = half(exp2((s - M)/ln 2) * 1/L) from the global max and sum, exactly as in the other attention kernels.
#pragma once

constexpr int AM_THREADS = 128;
constexpr int AM_WARPS = 4;
constexpr int AM_TK = 64;  // positions per staged tile

__device__ __forceinline__ void am_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void am_cp16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;  // 0 source bytes: zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
// apply_rotary_emb on one (even, odd) pair: x = (a, b), t = (cos, sin) -> (a*cos - b*sin, a*sin + b*cos), each fp16 op
// rounded once (jsgrad/models/llama.ts:17-32)
__device__ __forceinline__ uint32_t am_rope2(uint32_t xraw, uint32_t traw) {
  const __half2 x = *reinterpret_cast<const __half2*>(&xraw), t = *reinterpret_cast<const __half2*>(&traw);
  const __half xa = __low2half(x), xb = __high2half(x), co = __low2half(t), si = __high2half(t);
  const __half2 o = __halves2half2(hsub1(hmul1(xa, co), hmul1(xb, si)), hadd1(hmul1(xa, si), hmul1(xb, co)));
  return *reinterpret_cast<const uint32_t*>(&o);
}

template <int HD, int NREP>
__global__ void __launch_bounds__(AM_THREADS) attn_decode_mma_kernel(const AttnFusedArgs a) {
  constexpr int LD = HD + 8;      // padded tile row: fragment loads and ldmatrix rows fall on distinct banks
  constexpr int KS = HD / 16;     // k-steps of a score product
  constexpr int MT = HD / 16;     // 16-dim m-tiles of the output
  constexpr int MPW = (MT + AM_WARPS - 1) / AM_WARPS;
  constexpr int LPR = HD / 8;
  extern __shared__ __align__(16) float sc[];  // [NREP][chunk_cap] scores, later probabilities; then the K/V tiles
  __shared__ float red[AM_WARPS][8];
  __shared__ float s_m[NREP], s_l[NREP], s_M[NREP], s_rL[NREP];
  __shared__ float o_part[NREP * HD];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), CS = (int)cluster.num_blocks();
  const int g = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  __half* tiles = reinterpret_cast<__half*>(sc + (size_t)NREP * a.chunk_cap);  // [a.stages][AM_TK][LD]
  pdl_launch();
  pdl_wait();

  const int sq = a.seq ? a.seq[b] : b;
  if ((unsigned)sq >= (unsigned)a.n_seq) return;  // no such block-table row: skipped by every CTA of the cluster alike
  const int T = min(max(a.pos[b] + 1, 1), a.max_ctx);
  const int p = T - 1;  // position of the new token
  // positions per rank: a whole number of tiles, so that every tile starts on a multiple of AM_TK (the host sizes
  // chunk_cap to CS * (chunk_cap - 8) >= max_ctx rounded likewise)
  const int chunk = min(((T + CS - 1) / CS + AM_TK - 1) & ~(AM_TK - 1), a.chunk_cap - 8);
  const int t0 = min(rank * chunk, T), t1 = min(T, t0 + chunk);
  const int n_local = max(t1 - t0, 0);
  const int n_tiles = (n_local + AM_TK - 1) / AM_TK;
  const int32_t* bt_row = a.block_table + (size_t)sq * a.max_pages_per_seq;
  const __half* xrow = a.qkv + (size_t)b * a.qkv_stride;
  const __half* trow = a.table + (size_t)min(p, a.table_rows - 1) * HD;  // [hd/2][2] of position p

  // ---- the owner of position p rotates K and stores the new K / V rows
  if (!a.pre && t0 <= p && p < t1 && warp == 0 && lane < LPR) {
    const uint4 traw = ld_128(trow + lane * 8);
    const uint4 kraw = ld_128(xrow + (size_t)(a.H + g) * HD + lane * 8);
    const uint4 vraw = ld_128(xrow + (size_t)(a.H + a.G + g) * HD + lane * 8);
    const int pg = bt_row[p >> a.page_shift], slot = p & (a.page - 1);
    const size_t off = (((size_t)pg * a.G + g) * a.page + slot) * HD + (size_t)lane * 8;
    *reinterpret_cast<uint4*>(a.k_layer + off) = rope8(kraw, traw);
    *reinterpret_cast<uint4*>(a.v_layer + off) = vraw;
  }
  // ---- B fragments of q^T: column n = lane/4 is query head g*NREP + n (clamped: columns >= NREP are never stored)
  uint32_t qf[KS][2];
  {
    const __half* qh = xrow + (size_t)(g * NREP + min(qr, NREP - 1)) * HD;
#pragma unroll
    for (int k = 0; k < KS; k++) {
      const int c0 = k * 16 + qc, c1 = c0 + 8;
      uint32_t x0 = *reinterpret_cast<const uint32_t*>(qh + c0), x1 = *reinterpret_cast<const uint32_t*>(qh + c1);
      if (!a.pre) {
        x0 = am_rope2(x0, *reinterpret_cast<const uint32_t*>(trow + c0));
        x1 = am_rope2(x1, *reinterpret_cast<const uint32_t*>(trow + c1));
      }
      qf[k][0] = x0; qf[k][1] = x1;
    }
  }
  __syncthreads();  // the new K / V rows are visible to this CTA's loads below

  // A tile starts on a multiple of AM_TK, so with pages of AM_TK or more positions its rows lie back to back in one
  // page: one block-table lookup per tile and constant strides between a thread's copies.  Smaller pages take the
  // row-by-row path.
  const bool one_page = a.page >= AM_TK;
  auto load_tile = [&](const __half* layer, int j, __half* dst) {
    if (one_page) {
      const int ts = t0 + j * AM_TK, n_valid = t1 - ts;
      const __half* src = kv_row(layer, bt_row, ts, g, a.G, a.page, a.page_shift, HD) + tid * 8;
      __half* d = dst + (tid / (HD / 8)) * LD + (tid % (HD / 8)) * 8;
      constexpr int RPP = AM_THREADS / (HD / 8);  // rows per pass of the CTA
      if (n_valid >= AM_TK) {  // a whole tile (all but a rank's last): no per-row tests
        const uint32_t ds = (uint32_t)__cvta_generic_to_shared(d);
#pragma unroll
        for (int i = 0; i < AM_TK / RPP; i++)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ds + i * RPP * LD * 2), "l"(src + i * AM_THREADS * 8)
                       : "memory");
        return;
      }
#pragma unroll
      for (int i = 0; i < AM_TK / RPP; i++) {
        const bool ok = tid / (HD / 8) + i * RPP < n_valid;
        am_cp16(d + i * RPP * LD, ok ? src + i * AM_THREADS * 8 : layer, ok);
      }
      return;
    }
    for (int idx = tid; idx < AM_TK * (HD / 8); idx += AM_THREADS) {
      const int row = idx / (HD / 8), c = idx % (HD / 8);
      const int t = t0 + j * AM_TK + row;
      const bool ok = t < t1;
      const __half* src = ok ? kv_row(layer, bt_row, t, g, a.G, a.page, a.page_shift, HD) + c * 8 : layer;
      am_cp16(dst + row * LD + c * 8, src, ok);
    }
  };
  // The tiles travel through a ring of a.stages buffers, a.stages - 1 of them in flight while one is read.  Every
  // iteration commits exactly one group (an empty one past the last tile), so "all but the newest a.stages - 1 groups
  // have landed" always names the tile about to be read.
  const int S = a.stages;
  auto stage = [&](const __half* layer, int j) {
    if (j < n_tiles) load_tile(layer, j, tiles + (j % S) * AM_TK * LD);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto landed = [&]() {
    if (S == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else if (S == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else asm volatile("cp.async.wait_group 3;" ::: "memory");
  };

  // ---- scores of this rank's positions -> shared memory; warp w takes positions [16w, 16w+16) of every tile
  float lmax0 = -INFINITY, lmax1 = -INFINITY;  // heads qc and qc+1
  float* const srow = sc + min(qc, NREP - 1) * a.chunk_cap + warp * 16 + qr;  // head qc, this lane's first row of tile 0
  for (int j = 0; j < S - 1; j++) stage(a.k_layer, j);
#pragma unroll 1
  for (int j = 0; j < n_tiles; j++) {
    stage(a.k_layer, j + S - 1);  // into the buffer that iteration j - 1 read
    landed();
    __syncthreads();
    // A fragments of the warp's 16 positions: four 8x8 blocks per k-step in one ldmatrix; lane l names row
    // l%8 + 8*((l/8)%2) at dims 8*(l/16)
    const uint32_t ks = (uint32_t)__cvta_generic_to_shared(
        tiles + (j % S) * AM_TK * LD + (warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * LD + ((lane >> 4) << 3));
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < KS; k++) {
      uint32_t a0, a1, a2, a3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                   : "r"(ks + k * 32));
      am_mma(c, a0, a1, a2, a3, qf[k][0], qf[k][1]);
    }
    const int ia = j * AM_TK + warp * 16 + qr, ib = ia + 8;  // local positions of this lane's two rows
    if ((j + 1) * AM_TK <= n_local) {  // a whole tile
      float* s0 = srow + j * AM_TK;
      if (qc < NREP) {
        const float x = __fmul_rn(c[0], a.scale), y = __fmul_rn(c[2], a.scale);
        s0[0] = x; s0[8] = y; lmax0 = fmaxf(lmax0, fmaxf(x, y));
      }
      if (qc + 1 < NREP) {
        const float x = __fmul_rn(c[1], a.scale), y = __fmul_rn(c[3], a.scale);
        s0[a.chunk_cap] = x; s0[a.chunk_cap + 8] = y; lmax1 = fmaxf(lmax1, fmaxf(x, y));
      }
      __syncthreads();
      continue;
    }
    if (qc < NREP) {
      if (ia < n_local) { const float s = __fmul_rn(c[0], a.scale); sc[(size_t)qc * a.chunk_cap + ia] = s; lmax0 = fmaxf(lmax0, s); }
      if (ib < n_local) { const float s = __fmul_rn(c[2], a.scale); sc[(size_t)qc * a.chunk_cap + ib] = s; lmax0 = fmaxf(lmax0, s); }
    }
    if (qc + 1 < NREP) {
      if (ia < n_local) { const float s = __fmul_rn(c[1], a.scale); sc[(size_t)(qc + 1) * a.chunk_cap + ia] = s; lmax1 = fmaxf(lmax1, s); }
      if (ib < n_local) { const float s = __fmul_rn(c[3], a.scale); sc[(size_t)(qc + 1) * a.chunk_cap + ib] = s; lmax1 = fmaxf(lmax1, s); }
    }
    __syncthreads();  // the buffer read here is refilled by the next iteration
  }
  // the first V tiles travel while the statistics are worked out
  for (int j = 0; j < S - 1; j++) stage(a.v_layer, j);
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    lmax0 = fmaxf(lmax0, __shfl_xor_sync(0xffffffffu, lmax0, o));
    lmax1 = fmaxf(lmax1, __shfl_xor_sync(0xffffffffu, lmax1, o));
  }
  if (lane < 4) { red[warp][qc] = lmax0; red[warp][qc + 1] = lmax1; }
  __syncthreads();
  if (tid < NREP) {
    float m = red[0][tid];
    for (int w = 1; w < AM_WARPS; w++) m = fmaxf(m, red[w][tid]);
    s_m[tid] = m;
  }
  cluster.sync();  // every rank's max is published (a rank without positions publishes -inf)
  if (tid < NREP) {
    float M = -INFINITY;
    for (int rk = 0; rk < CS; rk++) M = fmaxf(M, *cluster.map_shared_rank(&s_m[tid], rk));
    s_M[tid] = M;
  }
  __syncthreads();
  // ---- e = exp2((s - M)/ln 2) against the global max, kept in place of the score, and this rank's sum of them
  const float log2e = 1.4426950408889634f;
  float lsum[NREP];
#pragma unroll
  for (int r = 0; r < NREP; r++) lsum[r] = 0.f;
  for (int t = tid; t < n_local; t += AM_THREADS) {
#pragma unroll
    for (int r = 0; r < NREP; r++) {
      float* sp = sc + r * a.chunk_cap + t;
      const float e = jg_xexp2_f32(__fmul_rn(__fsub_rn(*sp, s_M[r]), log2e));
      *sp = e;
      lsum[r] = __fadd_rn(lsum[r], e);
    }
  }
#pragma unroll
  for (int r = 0; r < NREP; r++) {
    const float v = warp_sum(lsum[r]);
    if (lane == 0) red[warp][r] = v;  // `red` was last read before the cluster barrier above
  }
  __syncthreads();
  if (tid < NREP) {
    float v = 0.f;
    for (int w = 0; w < AM_WARPS; w++) v += red[w][tid];
    s_l[tid] = v;
  }
  cluster.sync();
  // ---- normaliser L = the ranks' sums added in rank order
  if (tid < NREP) {
    float L = 0.f;
    for (int rk = 0; rk < CS; rk++) L = __fadd_rn(L, *cluster.map_shared_rank(&s_l[tid], rk));
    s_rL[tid] = __fdiv_rn(1.0f, L);
  }
  __syncthreads();
  // ---- probabilities p = half(e * 1/L), written as fp16 over the front half of each score row (zero
  // up to the end of the last tile).  The halves of positions [128i, 128i+128) land on the floats of positions
  // [64i, 64i+64), all of which every thread has read once the barrier of round i is passed.
  const int n_pad = n_tiles * AM_TK;
  for (int base = 0; base < n_pad; base += AM_THREADS) {
    const int t = base + tid;
    __half ph[NREP];
#pragma unroll
    for (int r = 0; r < NREP; r++) {
      const float e = t < n_local ? sc[r * a.chunk_cap + t] : 0.f;
      ph[r] = __float2half_rn(__fmul_rn(e, s_rL[r]));
    }
    __syncthreads();
    if (t < n_pad) {
#pragma unroll
      for (int r = 0; r < NREP; r++) reinterpret_cast<__half*>(sc + (size_t)r * a.chunk_cap)[t] = ph[r];
    }
  }
  __syncthreads();

  // ---- out^T = V^T . p^T: warp w owns output dims [16 * MPW * w, +16 * MPW)
  float acc[MPW][4];
#pragma unroll
  for (int m = 0; m < MPW; m++) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
  // B column n = lane/4 is head n (clamped); the lane's elements of a k-step are positions qc, qc+1 and qc+8, qc+9
  const __half* prow = reinterpret_cast<const __half*>(sc + (size_t)min(qr, NREP - 1) * a.chunk_cap) + qc;
#pragma unroll 1
  for (int j = 0; j < n_tiles; j++) {
    stage(a.v_layer, j + S - 1);
    landed();
    __syncthreads();
    const __half* Vs = tiles + (j % S) * AM_TK * LD;
    if (warp * MPW < MT) {
#pragma unroll
      for (int kk = 0; kk < AM_TK / 16; kk++) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(prow + j * AM_TK + kk * 16);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(prow + j * AM_TK + kk * 16 + 8);
#pragma unroll
        for (int m = 0; m < MPW; m++) {
          const int mt = warp * MPW + m;
          // V^T fragment: four 8x8 blocks of the tile read transposed; lane l names row (position) kk*16 + 8*(l/16) +
          // l%8 at dims mt*16 + 8*((l/8)%2)
          const __half* vp = Vs + (kk * 16 + ((lane >> 4) << 3) + (lane & 7)) * LD + mt * 16 + (((lane >> 3) & 1) << 3);
          uint32_t a0, a1, a2, a3;
          const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vp);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                       : "r"(addr));
          am_mma(acc[m], a0, a1, a2, a3, b0, b1);
        }
      }
    }
    __syncthreads();
  }
  if (warp * MPW < MT) {
#pragma unroll
    for (int m = 0; m < MPW; m++) {
      const int d = (warp * MPW + m) * 16 + qr;
      if (qc < NREP) { o_part[qc * HD + d] = acc[m][0]; o_part[qc * HD + d + 8] = acc[m][2]; }
      if (qc + 1 < NREP) { o_part[(qc + 1) * HD + d] = acc[m][1]; o_part[(qc + 1) * HD + d + 8] = acc[m][3]; }
    }
  }
  cluster.sync();

  // ---- each rank folds its slice of the NREP*HD outputs over the ranks, in rank order
  const int per_rank = (NREP * HD + CS - 1) / CS;
  for (int k = tid; k < per_rank; k += AM_THREADS) {
    const int idx = rank * per_rank + k;
    if (idx < NREP * HD) {
      float s = 0.f;
      for (int rk = 0; rk < CS; rk++) s = __fadd_rn(s, *cluster.map_shared_rank(&o_part[idx], rk));
      a.out[(size_t)b * a.H * HD + (size_t)g * NREP * HD + idx] = __float2half_rn(s);
    }
  }
  cluster.sync();  // peers may still be reading this CTA's shared memory
}
