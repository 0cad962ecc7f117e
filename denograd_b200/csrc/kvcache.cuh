// The paged KV cache object shared by the attention kernels (decode in attention.cu, multi-position chunks in
// attention_chunk.cu).  The layout is private to the device: the reference keeps one contiguous
// [2][B][max_ctx][G][hd] tensor per layer (jsgrad/models/llama.ts:78-90); here pages of `page_size` positions are
// addressed through a block table.
#pragma once
#include "common.cuh"

struct jg_kvcache {
  jg_dev* dev;
  jg_kvcache_desc d;
  __half* k_pool;  // [L][n_pages][G][page][hd]
  __half* v_pool;
  int32_t* block_table;  // [max_batch][max_pages_per_seq]
  float* scores;         // [max_batch][H][max_ctx]
  float* part_ml;        // [max_batch][H][n_split][2]  (max, sum of exp relative to that max)
  float* part_o;         // [max_batch][H][n_split][hd]
  unsigned int* tickets; // [max_batch][G]
  int n_split;
  int max_ctx;
  size_t layer_elems;  // elements of one layer of K (or V)
  uint64_t bytes;
};

// Address of the K (or V) row of position t of kv head g for the sequence whose block-table row is bt_row.
__device__ __forceinline__ const __half* kv_row(const __half* layer, const int32_t* bt_row, int t, int g, int G,
                                                int page, int page_shift, int hd) {
  const int pg = bt_row[t >> page_shift];
  const int slot = t & (page - 1);
  return layer + (((size_t)pg * G + g) * page + slot) * hd;
}

// The same for a caller-owned pool of `n_pages` pages whose block table nobody validated: an entry outside the pool
// yields a null pointer, which the callers read as a row of zeros (what an unwritten cache position holds).
// n_pages = 0 means the table was validated on the host (jg_kvcache_set_block_table) and is followed as is.
__device__ __forceinline__ const __half* kv_row_checked(const __half* layer, const int32_t* bt_row, int t, int g, int G,
                                                        int page, int page_shift, int hd, int n_pages) {
  const int pg = bt_row[t >> page_shift];
  if (n_pages > 0 && (unsigned)pg >= (unsigned)n_pages) return nullptr;
  const int slot = t & (page - 1);
  return layer + (((size_t)pg * G + g) * page + slot) * hd;
}
__device__ __forceinline__ uint4 ld_kv_128(const __half* row, int off) {
  return row ? *reinterpret_cast<const uint4*>(row + off) : make_uint4(0, 0, 0, 0);
}

#ifdef __CUDACC__
// apply_rotary_emb on eight halves = four (re, im) pairs against four (cos, sin) pairs (jsgrad/models/llama.ts:23-32)
__device__ __forceinline__ uint4 rope8(const uint4& xraw, const uint4& traw) {
  const __half* x = reinterpret_cast<const __half*>(&xraw);
  const __half* t = reinterpret_cast<const __half*>(&traw);
  __align__(16) __half o[8];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const __half xa = x[2 * i], xb = x[2 * i + 1], co = t[2 * i], si = t[2 * i + 1];
    o[2 * i] = hsub1(hmul1(xa, co), hmul1(xb, si));
    o[2 * i + 1] = hadd1(hmul1(xa, si), hmul1(xb, co));
  }
  return *reinterpret_cast<uint4*>(o);
}
#endif

static inline int ilog2(int v) { int s = 0; while ((1 << s) < v) s++; return s; }
