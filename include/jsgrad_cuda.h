/*
 * jsgrad_cuda.h — C ABI of libjsgrad_cuda.so, the native half of a `CUDA` device for jsgrad.
 *
 * The TypeScript half (class CUDA extends Compiled, with its Allocator / Program / graph runner) binds exactly
 * these symbols through Deno.dlopen, the way jsgrad/runtime/ops_clang.ts:40-54 binds one generated C function
 * and dawn/bindings.ts binds libwebgpu_dawn.  Everything crosses the boundary as plain integers and pointers:
 *   - a device buffer is a uint64_t device address (the engine's opaque `Buf`); sub-buffers are address + offset;
 *   - host memory is a `const void*` / `void*` (Deno 'buffer' / 'pointer');
 *   - every function returns an int status: 0 on success, an errno-style code otherwise, with the message
 *     available from jg_last_error() (the TypeScript side turns a non-zero status into `throw new Error(...)`,
 *     the reference's own convention: jsgrad/runtime/ops_clang.ts:34-35,42).
 *
 * All kernels of one device are issued on that device's single stream, in call order (the engine awaits each
 * device call in program order: jsgrad/engine/realize.ts:215-218, jsgrad/engine/jit.ts:214).  Only
 * jg_copyout, jg_device_sync and jg_timer_stop block the calling thread.
 *
 * Built for sm_100a only.  There is no CPU fallback: if the library cannot open a CUDA device every entry point
 * fails with JG_EIO.
 */
#ifndef JSGRAD_CUDA_H
#define JSGRAD_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JG_OK 0
#define JG_EIO 5         /* a CUDA runtime call failed (message in jg_last_error) */
#define JG_ENOMEM 12     /* device or pinned-host allocation failed */
#define JG_EINVAL 22     /* rejected before any launch: bad pointer, size, alignment or unsupported shape */
#define JG_ENOTSUP 95    /* shape outside what the kernels implement */
#define JG_ETIMEDOUT 110 /* a bounded device-side wait gave up */

typedef struct jg_dev jg_dev;         /* one opened CUDA device + its stream */
typedef struct jg_graph jg_graph;     /* a captured, replayable list of launches */
typedef struct jg_kvcache jg_kvcache; /* paged K/V pool of one model on one device */
typedef struct jg_comm jg_comm;       /* tensor-parallel communicator of one rank */
typedef struct jg_step jg_step;       /* one model's decode step as a single persistent kernel */
typedef struct jg_program jg_program; /* one run-time compiled kernel loaded on one device */

/* ---- Compiled: jsgrad/runtime/allocator.ts:166-191 (ctor/init/synchronize), device lookup
 *      jsgrad/device.ts:26-35 (`new DEVICES['CUDA']('CUDA:3')`: the ordinal is parsed from the device name). */
typedef struct {
  char name[64];
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  uint64_t total_mem;
  uint64_t l2_bytes;
  int32_t max_smem_per_block;
} jg_props;

int jg_device_count(int32_t* out);
int jg_device_open(int32_t ordinal, jg_dev** out);
int jg_device_close(jg_dev* dev);
int jg_device_sync(jg_dev* dev);
int jg_device_props(jg_dev* dev, jg_props* out);
const char* jg_last_error(void);
/* Kernels launched by this library on `dev` since it was opened (launches replayed through a graph count each
 * time the graph runs).  Bookkeeping for DEBUG-style statistics, cf. GlobalCounters.kernel_count
 * (jsgrad/helpers/helpers.ts:556-563). */
int jg_launch_count(jg_dev* dev, uint64_t* out);

/* ---- Allocator: jsgrad/runtime/allocator.ts:28-47 (_alloc/_free/_copyin/_copyout/_offset/_transfer). */
int jg_alloc(jg_dev* dev, size_t nbytes, uint64_t* dptr);
int jg_free(jg_dev* dev, uint64_t dptr);
int jg_copyin(jg_dev* dev, uint64_t dst, const void* host, size_t nbytes);  /* host buffer reusable on return */
int jg_copyout(jg_dev* dev, void* host, uint64_t src, size_t nbytes);       /* synchronises the stream */
int jg_transfer(jg_dev* dst_dev, uint64_t dst, jg_dev* src_dev, uint64_t src, size_t nbytes); /* peer copy */
int jg_memset(jg_dev* dev, uint64_t dst, int32_t byte, size_t nbytes);
int jg_copy(jg_dev* dev, uint64_t dst, uint64_t src, size_t nbytes);  /* device-to-device on dev's stream */
/* Page-locked host staging (BufferSpec.host, jsgrad/runtime/allocator.ts:8-25): copies from/to it are truly
 * asynchronous. */
int jg_host_alloc(size_t nbytes, void** out);
int jg_host_free(void* p);
int jg_copyin_async(jg_dev* dev, uint64_t dst, const void* pinned_host, size_t nbytes);
int jg_copyout_async(jg_dev* dev, void* pinned_host, uint64_t src, size_t nbytes);

/* ---- Program.call(..., wait): jsgrad/runtime/allocator.ts:98-107, jsgrad/runtime/ops_clang.ts:51-53.
 *      `wait=true` is start -> calls -> stop; stop blocks and returns the elapsed device time in seconds. */
int jg_timer_start(jg_dev* dev);
int jg_timer_stop(jg_dev* dev, double* seconds);

/* ---- Compiler / Program for generated source: jsgrad/runtime/allocator.ts:98-107 (Program), :121-139 (CompileError,
 *      Compiler); the reference's own instance of the pair is jsgrad/runtime/ops_clang.ts:7-54.  The reference ships a
 *      CUDA code generator (CUDARenderer, jsgrad/renderer/cstyle.ts:348-419) and no CUDA runtime; these entry points are
 *      that runtime, for every scheduled AST the hand-written kernels below do not cover.
 *      jg_cuda_compile: Compiler.compile — CUDA C source -> cubin for `arch` (null or "" = "sm_100a") through NVRTC; needs
 *      no device; a source that does not compile is JG_EINVAL with the compiler's log in jg_last_error (CompileError).
 *      The image is released with jg_cuda_image_free (its bytes may be kept in the engine's compile cache and loaded
 *      again later).
 *      jg_program_load: Program.init(name, lib) — `name` is the kernel function (`extern "C" __global__`).
 *      jg_program_call: Program.call(bufs, {global_size, local_size, vals}) — the kernel receives every buffer as a
 *      device pointer, then every variable as a 32-bit int (ops_clang.ts:44-52); global_size / local_size point at
 *      three numbers each (null = 1, 1, 1) and become the grid and the block.  The launch is ordered on the device's
 *      stream with all other kernels, is recorded by a graph capture and timed by jg_timer_start / jg_timer_stop. */
int jg_cuda_compile(const char* src, const char* arch, uint8_t** image, uint64_t* size);
int jg_cuda_image_free(uint8_t* image);
int jg_program_load(jg_dev* dev, const char* name, const uint8_t* image, uint64_t size, jg_program** out);
int jg_program_call(jg_program* program, const uint64_t* bufs, int32_t n_bufs, const int32_t* vals, int32_t n_vals,
                    const uint32_t* global_size, const uint32_t* local_size);
int jg_program_destroy(jg_program* program);

/* ---- Compiled.graph / GraphRunner: jsgrad/engine/jit.ts:14-144 (batching of a captured kernel list) and
 *      CapturedJit replay jsgrad/engine/jit.ts:190-217.  Between begin and end every launch on `dev` is recorded
 *      instead of executed; launch replays the list.  Values that change between replays (tokens, positions —
 *      the jit's `start_pos` Variable, jsgrad/models/llama.ts:217) live in device memory and are read by the
 *      kernels at run time, so a replay needs no patching. */
int jg_graph_begin(jg_dev* dev);
int jg_graph_end(jg_dev* dev, jg_graph** out);
int jg_graph_launch(jg_dev* dev, jg_graph* g);
int jg_graph_destroy(jg_graph* g);

/* ---- Kernels.  Shapes: M = rows of activations (batch x new tokens), weights are [N][K] row-major
 *      (nn.Linear layout, jsgrad/nn/index.ts:403-412).  `scale` = 0 selects fp16 weights; otherwise `w` is int8
 *      and `scale` is the fp16 per-output-row scale of Int8Linear (jsgrad/models/llama3.ts:27-35).
 *      All activation tensors are fp16, densely packed. */

/* Embedding.call / Int8Embedding.call: jsgrad/nn/index.ts:607-619, jsgrad/models/llama3.ts:71-77.
 * tokens: int32[n_tok] in device memory. */
int jg_embed(jg_dev* dev, uint64_t out, uint64_t tokens, uint64_t w, uint64_t scale, int32_t n_tok, int32_t dim,
             int32_t vocab);

/* RMSNorm.call: jsgrad/nn/index.ts:586-588. */
int jg_rmsnorm(jg_dev* dev, uint64_t y, uint64_t x, uint64_t w, int32_t rows, int32_t dim, float eps);

/* Linear.call / Int8Linear.call: jsgrad/nn/index.ts:411, jsgrad/models/llama3.ts:35; `residual` (0 = none) is
 * the `x.add(...)` of TransformerBlock.call, jsgrad/models/llama.ts:125-126, fused as an epilogue.
 * Row counts: 1-2 rows of fp16 weights stream through the CUDA cores (norm fused where the entry point has one).
 * From 3 rows on, and for int8 weights at every row count, the tensor cores take over and the fused-norm entry
 * points want norm_w = 0 with rows normalised by jg_rmsnorm first: fp16 weights with N % 128 == 0 and K % 64 == 0 on
 * the tcgen05 kernel (any M), other fp16 shapes and int8 weights on the mma.sync kernel (M <= 64; more rows are
 * JG_ENOTSUP: split them into chunks of 64, or for int8 use jg_dequant_i8_f16 and project over the fp16 copy). */
int jg_linear(jg_dev* dev, uint64_t y, uint64_t x, uint64_t w, uint64_t scale, uint64_t residual, int32_t M,
              int32_t N, int32_t K);

/* RMSNorm followed by Linear on the same rows (attention_norm -> wq|wk|wv, ffn_norm -> w1/w3, norm -> output:
 * jsgrad/models/llama.ts:125-126,210) as one kernel; the norm is over K. */
int jg_norm_linear(jg_dev* dev, uint64_t y, uint64_t x, uint64_t norm_w, float eps, uint64_t w, uint64_t scale,
                   int32_t M, int32_t N, int32_t K);

/* FeedForward.call up to the elementwise product: y = silu(norm(x) W1^T) * (norm(x) W3^T),
 * jsgrad/models/llama.ts:108-110 + jsgrad/tensor.ts:2909-2911,3210-3226.  norm_w = 0 skips the norm. */
int jg_norm_swiglu(jg_dev* dev, uint64_t y, uint64_t x, uint64_t norm_w, float eps, uint64_t w_gate,
                   uint64_t s_gate, uint64_t w_up, uint64_t s_up, int32_t M, int32_t N, int32_t K);

/* Elementwise silu(g) * u on already-computed projections (same source lines). */
int jg_swiglu(jg_dev* dev, uint64_t y, uint64_t g, uint64_t u, int64_t n);

/* Final norm + output projection for M rows + greedy selection: writes the fp16 logits [M][V] and folds
 * (value, lowest index) into key[M] (uint64 each, must be zero on entry); jg_argmax_finalize turns the keys into
 * int32 token ids and re-zeroes them.  jsgrad/models/llama.ts:210-212,137; jsgrad/tensor.ts:2314-2320.
 * norm_w = 0 skips the norm (rows already normalised). */
int jg_norm_logits_argmax(jg_dev* dev, uint64_t logits, uint64_t key, uint64_t x, uint64_t norm_w, float eps,
                          uint64_t w, uint64_t scale, int32_t M, int32_t V, int32_t K);
int jg_argmax_finalize(jg_dev* dev, uint64_t tokens_out, uint64_t key, int32_t M);
/* Tensor.argmax over the last axis of fp16 [rows][n]: jsgrad/tensor.ts:2314-2320. */
int jg_argmax(jg_dev* dev, uint64_t out_idx, uint64_t x, int32_t rows, int32_t n);

/* `sample` beyond its greedy branch (jsgrad/models/llama.ts:131-185): alpha penalties (:142-147), NaN -> -inf, softmax
 * of logits / temp (:150-153), k rounds of largest-probability-with-lowest-index (:160-167), the approximate top-p cut
 * on those k (:171-173) and the multinomial draw (:176-179; Tensor.multinomial, jsgrad/tensor.ts:1164-1172).  The draw
 * needs one uniform sample in [0, 1) per row, u[B] (float32, device) — what Tensor.rand delivers in the reference; the
 * caller supplies it.  logits: fp16 [B][V] (widened to fp32 as jsgrad/models/llama.ts:210 does); tokens_out: int32 [B];
 * alpha_counter: int32 [B][V] (the reference's module-level counter, zero-initialised by the caller; incremented at
 * the chosen token) or 0 when af = ap = 0.  k = 0 draws from the whole distribution; k <= 512.  temp >= 1e-6 (below
 * that `sample` is jg_argmax).  Every float32 sum is added in the order the reference's kernels add it, so the token
 * is a function of (logits, u) only. */
int jg_sample(jg_dev* dev, uint64_t tokens_out, uint64_t logits, uint64_t u, uint64_t alpha_counter, int32_t B, int32_t V,
              float temp, int32_t k, float p, float af, float ap);

/* precompute_freqs_cis cast to fp16: jsgrad/models/llama.ts:10-14,205. table: fp16 [end][head_dim/2][2]. */
int jg_freqs_cis(jg_dev* dev, uint64_t table, int32_t head_dim, int32_t end, double theta);

/* ---- KV cache (Attention.cache_kv, jsgrad/models/llama.ts:78-90) held as a paged pool: per layer
 *      K and V are [n_pages][n_kv_heads][page_size][head_dim] fp16; block_table[b][i] names the page holding
 *      positions [i*page_size, (i+1)*page_size) of batch row b.  The layout is private to the device. */
typedef struct {
  int32_t n_layers, n_kv_heads, head_dim;
  int32_t page_size;      /* tokens per page: 16, 32 or 64 */
  int32_t n_pages;        /* pages in the pool (shared by all batch rows) */
  int32_t max_batch;
  int32_t max_pages_per_seq;
  int32_t n_heads;        /* query heads served by this cache (sizes the attention scratch) */
  int32_t n_split;        /* context splits per (batch row, kv head) in decode attention; 0 = choose */
} jg_kvcache_desc;

int jg_kvcache_create(jg_dev* dev, const jg_kvcache_desc* desc, jg_kvcache** out);
int jg_kvcache_destroy(jg_kvcache* kv);
/* host int32 [max_batch][max_pages_per_seq]; the default after create is the identity mapping
 * (row b owns pages b*max_pages_per_seq ...). */
int jg_kvcache_set_block_table(jg_kvcache* kv, const int32_t* table);
int jg_kvcache_bytes(jg_kvcache* kv, uint64_t* out);

/* apply_rotary_emb on Q and K + cache assignment (jsgrad/models/llama.ts:23-32,87) for S=1 rows:
 * qkv: fp16 [B][(H + 2G) * hd] = wq|wk|wv outputs; Q is rotated in place, rotated K and V go to the cache at
 * position pos[b] (device int32[B], the `start_pos` variable).  table: [table_rows][hd/2][2] from jg_freqs_cis;
 * a row whose position lies outside the table or the cache is skipped. */
int jg_rope_kvwrite(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t qkv, uint64_t table, int32_t table_rows,
                    uint64_t pos, int32_t B, int32_t H);

/* scaled_dot_product_attention for one new token per row over positions [0, pos[b]] with repeat_kv head
 * sharing (jsgrad/tensor.ts:3920-3934,2186-2214; jsgrad/models/llama.ts:34-39,89-96).
 * q is read from qkv ([B][(H+2G)*hd], first H*hd of each row); out: fp16 [B][H*hd]. */
int jg_attn_decode(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t pos,
                   int32_t B, int32_t H);

/* The three steps above for one new token per row in a single launch: rotate Q and K (jsgrad/models/llama.ts:23-32),
 * store K/V at pos[b] (:87), attend over [0, pos[b]] (jsgrad/tensor.ts:3920-3934).  A thread-block cluster shares one
 * (row, kv head) and exchanges the softmax statistics through distributed shared memory, so no scratch memory is
 * used; the per-CTA slice of the context must fit in shared memory (JG_ENOTSUP otherwise — use the two calls above).
 * Unlike jg_rope_kvwrite this leaves the Q slice of `qkv` unrotated. */
int jg_attn_decode_fused(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t table,
                         int32_t table_rows, uint64_t pos, int32_t B, int32_t H);

/* Several new positions per sequence in one call (Transformer.forward with S > 1, jsgrad/models/llama.ts:201-213: the
 * additive causal mask of :208 lets row (b, s) see positions [0, start_pos + s]).  Rows are independent: row r has
 * position pos[r] and belongs to sequence seq[r] (its block-table row).  jg_rope_kvwrite_rows rotates Q/K of all rows
 * and stores K/V; jg_attn_rows then attends row r over [0, pos[r]] of its sequence — which includes the rows of the
 * same call that precede it, as the mask prescribes.  R is not limited by the cache's max_batch. */
int jg_rope_kvwrite_rows(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t qkv, uint64_t table, int32_t table_rows,
                         uint64_t pos, uint64_t seq, int32_t R, int32_t H);
int jg_attn_rows(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t pos, uint64_t seq,
                 int32_t R, int32_t H);

/* The same attention for a regular chunk, on the tensor cores: Sc consecutive positions of each of B sequences, rows
 * laid out position-major (row = s * B + b) with pos[s * B + b] = pos[b] + s; seq[b] names the block-table row of
 * sequence b (0 = row b).  K and V of the chunk must already be in the cache (jg_rope_kvwrite_rows) and Q rotated.
 * Same result as jg_attn_rows up to the summation order of the fp32 accumulations. */
int jg_attn_chunk(jg_dev* dev, jg_kvcache* kv, int32_t layer, uint64_t out, uint64_t qkv, uint64_t pos, uint64_t seq,
                  int32_t B, int32_t Sc, int32_t H);

/* The whole decode step — embedding, every TransformerBlock, final norm, output projection and greedy pick
 * (Transformer.forward for one token per row, jsgrad/models/llama.ts:201-220) — as ONE persistent cooperative kernel:
 * what the reference replays as a captured batch of kernels (TinyJit / GraphRunner, jsgrad/engine/jit.ts:71-141,
 * 273-353).  One CTA per SM stays resident; the former kernels are phases separated by grid-wide barriers, and the
 * first weights of the next projection are already in flight when a CTA arrives at a barrier, so the HBM stream does
 * not drain at every kernel boundary.  fp16 weights, 1 or 2 rows, head_dim 64 / 128 with up to 4 query heads per kv
 * head, n_heads * head_dim == dim; other shapes: JG_ENOTSUP (the caller keeps the launch-per-op path).
 * Tensor parallelism (`comm` set; every rank makes the same calls): the dimensions are the rank's shares as
 * Llama3's shard plan cuts them (jsgrad/models/llama3.ts:239-249: wq|wk|wv and w1 / w3 by rows, wo and w2 by
 * columns, `output` by vocabulary rows; n_heads and the cache's kv heads are the rank's); the partial sums of wo and
 * w2 and the ranks' best (value, index) keys cross NVLink as flag-in-data entries inside the kernel, every wait
 * bounded by the communicator's limit.
 * `layers` is a HOST pointer to n_layers x 7 device addresses: attention_norm.weight, wq|wk|wv (one allocation),
 * wo, ffn_norm.weight, w1, w3, w2.  The cache object supplies the K/V pools and the block table (identity row map). */
typedef struct jg_step_desc {
  int32_t n_layers;
  int32_t dim;
  int32_t hidden_dim;
  int32_t n_heads;
  int32_t vocab_size;
  int32_t freqs_rows;      /* rows of the RoPE table */
  float norm_eps;
  int32_t vocab_offset;    /* tensor parallelism: vocabulary index of row 0 of `output` (0 on one GPU) */
  uint64_t layers;         /* host pointer, see above */
  uint64_t tok_embeddings; /* fp16 [vocab][dim] */
  uint64_t out_norm;       /* fp16 [dim] */
  uint64_t output;         /* fp16 [vocab][dim] */
  uint64_t freqs_cis;      /* fp16 [freqs_rows][head_dim/2][2] from jg_freqs_cis */
  uint64_t comm;           /* tensor parallelism: the rank's jg_comm* with its peer buffers open; 0 on one GPU */
  int64_t embed_rows;      /* rows of tok_embeddings (the whole vocabulary on every rank); 0 = vocab_size */
} jg_step_desc;
int jg_step_create(jg_dev* dev, jg_kvcache* kv, const jg_step_desc* desc, jg_step** out);
int jg_step_destroy(jg_step* step);
/* n_steps decode steps for B rows.  tokens / pos: device int32 [B] (pos = index of the new token); h, qkv, attn, ffn:
 * the step's activation buffers ([B][dim], [B][(H+2G)*hd], [B][dim], [B][hidden] fp16); logits: fp16 [B][vocab] of
 * the last step; next_tokens: int32 [n_steps][B].  With `advance` the picks are fed back
 * (tokens <- pick, pos += 1) between steps and stored to tokens / pos at the end; n_steps > 1 requires it.
 * Every wait on another CTA is bounded (JG_STEP_TIMEOUT_MS, default 2000): a launch whose CTAs are not all making
 * progress ends with JG_ETIMEDOUT at the next synchronising call. */
int jg_step_run(jg_step* step, uint64_t tokens, uint64_t pos, uint64_t h, uint64_t qkv, uint64_t attn, uint64_t ffn,
                uint64_t logits, uint64_t next_tokens, int32_t B, int32_t n_steps, int32_t advance);

/* jg_attn_decode without any allocation by the library.  It has no counterpart in the reference; it exists for hosts
 * that must keep a kernel library from allocating device memory: an engine whose allocator owns the whole device and
 * places every buffer itself (jsgrad's memory planner / LRU allocator), or a loop that cannot take the device-wide
 * synchronisation of cudaMalloc / cudaFree.  The caller passes every input and output: the layer's K and V pools
 * ([n_pages][G][page_size][head_dim] fp16), the int32 block table [B][max_pages_per_seq], pos[B], qkv and out as in
 * jg_attn_decode (Q already rotated, K/V already stored), and n_pages, the number of pages the two pools hold: the
 * block table is the caller's and nobody validated it, so an entry outside [0, n_pages) is not followed — that
 * position reads as a row of zeros, like an unwritten one.  Scores, split statistics and partial outputs live in a
 * fixed 8 MiB array inside the library image (held by every GPU that loads the library, until the process exits);
 * shapes that need more are rejected with JG_EINVAL:
 *     4*B*H*(max_pages_per_seq*page_size) + 4*B*H*n_split*(2 + head_dim) + 4*B*G  bytes (each part rounded to 256).
 * The first call on a device looks up the array's device address; make that call before any stream capture begins
 * (a first call made during jg_graph_begin .. jg_graph_end is rejected with JG_EINVAL).
 * All calls share the array, which keeps the previous call's contents (the call clears the part that must start at
 * zero): two calls that overlap on the GPU — different streams, or different devices' handles on one GPU — race. */
int jg_attn_decode_noalloc(jg_dev* dev, uint64_t out, uint64_t qkv, uint64_t k_layer, uint64_t v_layer,
                           uint64_t block_table, uint64_t pos, int32_t B, int32_t H, int32_t G, int32_t head_dim,
                           int32_t page_size, int32_t max_pages_per_seq, int32_t n_split, int32_t n_pages);

/* pos[b] += 1 for b < B (the host-side `start_pos++` of the decode loop, jsgrad/models/llama3.ts:284-295,
 * kept on the device so a captured step can be replayed without host input). */
int jg_pos_advance(jg_dev* dev, uint64_t pos, int32_t B);

/* ---- Tensor parallelism.  The reference only declares a sharding plan (jsgrad/models/llama3.ts:239-249; its
 *      jsgrad/multi.ts is a stub whose functions all throw), so these have no executable counterpart there.  One rank =
 *      one process = one jg_dev.  Column-parallel projections (wq/wk/wv by heads, w1/w3, vocabulary-sharded output)
 *      need no exchange; row-parallel ones (wo, w2) produce fp32 partial sums that are all-reduced before the single
 *      rounding to fp16 and the residual add. */
int jg_comm_unique_id(const char* nccl_path, void* id128);  /* rank 0 makes the 128-byte id; share it out of band */
int jg_comm_init(jg_dev* dev, const char* nccl_path, const void* id128, int32_t rank, int32_t world, jg_comm** out);
int jg_comm_destroy(jg_comm* comm);
int jg_allreduce_sum_f32(jg_comm* comm, uint64_t buf, uint64_t count);  /* in place, on the device's stream */
int jg_allreduce_max_u64(jg_comm* comm, uint64_t buf, uint64_t count);  /* greedy keys of a sharded vocabulary */
/* The same two exchanges as one kernel per rank over NVLink peer memory, for the small messages of a decode step
 * (multi.ts has no counterpart: its functions throw).  jg_comm_peer_export allocates this rank's exchange buffer and
 * returns its 64-byte CUDA IPC handle; after every rank's handle has been gathered out of band (world x 64 bytes in
 * rank order) jg_comm_peer_open maps the peers' buffers.  jg_peer_allreduce_residual then does
 * h[i] <- h[i] + half(sum over ranks of part32[i]) in one launch: each partial sum is stored, paired with the number
 * of the exchange, into every peer's buffer with one 8-byte store; the peers' entries are awaited on this rank's own
 * buffer (bounded: JG_ETIMEDOUT at the next synchronisation if a peer never arrives; JG_PEER_TIMEOUT_MS, default
 * 5000) and added in rank order.  All ranks must issue the same sequence of peer reductions.
 * jg_comm_peer_capacity reports the largest n (0 while the peer path is not open). */
int jg_comm_peer_export(jg_comm* comm, void* handle64);
int jg_comm_peer_open(jg_comm* comm, const void* handles);
int jg_comm_peer_capacity(jg_comm* comm, uint64_t* floats);
int jg_peer_allreduce_residual(jg_comm* comm, uint64_t h, uint64_t part32, uint64_t n);
int jg_peer_allreduce_max_u64(jg_comm* comm, uint64_t keys, uint64_t n);
/* A row-parallel Linear (this rank holds a K-slice of W, nn/index.ts:411) fused with that exchange and the residual
 * add: h <- h + half(sum over ranks of x . W^T) in one launch per rank, for up to 8 rows.  CTA c of every rank owns
 * the same output rows: it stores its partial sums, each paired with the exchange number, into the peers' buffers,
 * waits (bounded) for the peers' entries of its rows and finishes them. */
int jg_linear_allreduce_residual(jg_comm* comm, uint64_t h, uint64_t x, uint64_t w, uint64_t scale, int32_t M, int32_t N,
                                 int32_t K);
/* The same all-reduce cut in two so that no kernel sits waiting for another rank (up to 8 rows, M * N <= 32768):
 * jg_tp_linear_push is the row-parallel Linear whose epilogue stores the partial sums into every rank's buffer and
 * returns at once; the projection that consumes the sum — the next RMSNorm + Linear of the block
 * (jsgrad/models/llama.ts:125-126: ffn_norm -> w1/w3 after wo, the next block's attention_norm -> wq|wk|wv after w2,
 * norm -> output after the last block, :210) — adds the ranks' entries in rank order in its prologue (bounded wait),
 * rounds once, adds the residual stream h_in and leaves the new stream in h_out (a different buffer), then normalises
 * and projects as jg_norm_linear / jg_norm_swiglu / jg_norm_logits_argmax_shard do.  Every push must be followed, on
 * every rank, by exactly one of the three consuming calls (same M, K = the push's N) before any other exchange. */
int jg_tp_linear_push(jg_comm* comm, uint64_t x, uint64_t w, uint64_t scale, int32_t M, int32_t N, int32_t K);
int jg_tp_norm_linear(jg_comm* comm, uint64_t y, uint64_t h_out, uint64_t h_in, uint64_t norm_w, float eps, uint64_t w,
                      uint64_t scale, int32_t M, int32_t N, int32_t K);
int jg_tp_norm_swiglu(jg_comm* comm, uint64_t y, uint64_t h_out, uint64_t h_in, uint64_t norm_w, float eps, uint64_t w_gate,
                      uint64_t s_gate, uint64_t w_up, uint64_t s_up, int32_t M, int32_t N, int32_t K);
int jg_tp_norm_logits_argmax(jg_comm* comm, uint64_t logits, uint64_t key, uint64_t h_out, uint64_t h_in, uint64_t norm_w,
                             float eps, uint64_t w, uint64_t scale, int32_t M, int32_t V_local, int32_t K,
                             int32_t row_offset);
/* Larger sums (a batch of decode rows, a short prompt chunk; n <= 262144 values, n % 4 == 0) as a two-shot exchange:
 * jg_linear_partial writes this rank's fp32 partial sums into the region jg_comm_peer_partial names (part of the
 * exchange buffer, readable by the peers); jg_peer_allreduce2_residual then has each rank add 1/world of the values
 * over all ranks (plain peer loads, rank order), round, add the residual and send the finished fp16 values to every
 * peer: h[i] <- h[i] + half(sum over ranks of partial[i]). */
int jg_comm_peer_partial(jg_comm* comm, uint64_t* ptr, uint64_t* floats);
int jg_peer_allreduce2_residual(jg_comm* comm, uint64_t h, uint64_t n);
/* All ranks in ONE process, the reference engine's own threading model (one JS thread drives every device:
 * Tensor.shard, jsgrad/tensor.ts:676-687; jsgrad/models/llama3.ts:239-249): devs[r] becomes rank r, out[r] its
 * communicator.  The exchange buffers are addressed directly (cudaDeviceEnablePeerAccess), so no id and no handles
 * are exchanged and jg_comm_peer_export / _open are not used.  NCCL collectives issued for several ranks by one
 * thread must be bracketed by jg_comm_group_begin / jg_comm_group_end (ncclGroupStart / ncclGroupEnd). */
int jg_comm_init_all(int32_t n, jg_dev** devs, const char* nccl_path, jg_comm** out);
int jg_comm_group_begin(void);
int jg_comm_group_end(void);
/* y32[m][n] = sum_k x[m][k] W[n][k] left in fp32 (this rank's K-slice of a row-parallel Linear, nn/index.ts:411). */
int jg_linear_partial(jg_dev* dev, uint64_t y32, uint64_t x, uint64_t w, uint64_t scale, int32_t M, int32_t N, int32_t K);
/* h <- h + half(p32): rounding + residual add of jsgrad/models/llama.ts:125-126 after the all-reduce. */
int jg_residual_add_f32(jg_dev* dev, uint64_t h, uint64_t p32, int64_t n);
/* jg_norm_logits_argmax over rows [row_offset, row_offset + V_local) of the output matrix: keys carry global ids. */
int jg_norm_logits_argmax_shard(jg_dev* dev, uint64_t logits, uint64_t key, uint64_t x, uint64_t norm_w, float eps,
                                uint64_t w, uint64_t scale, int32_t M, int32_t V_local, int32_t K, int32_t row_offset);

/* Int8Linear's dequantised matrix (jsgrad/models/llama3.ts:35: weight.cast(half) * scale, fp16 [N][K]) written out
 * once, so that a call with many rows can use the fp16 tensor-core projection on it.
 * Weights written on the device: the tensor-core projections start loading weight tiles while the preceding launch
 * is still draining.  The library remembers the destinations of its own last 16 device-side writes since the stream
 * was last synchronised (this function, the jg_fill_* family, jg_linear / jg_norm_linear outputs, jg_copy, jg_memset,
 * jg_copyin_async) and holds those loads back when a weight pointer falls inside one of them.  A matrix written in
 * any other way (another stream, more than 16 launches ago without a synchronisation in between) needs a
 * jg_device_sync before it is used as `w`. */
int jg_dequant_i8_f16(jg_dev* dev, uint64_t dst, uint64_t w, uint64_t scale, int64_t N, int64_t K);

/* NF4Linear's dequantised matrix (jsgrad/models/llama3.ts:79-94): element i of the flattened [out][in] matrix is
 * half(CODE[code_i] * scale[i / block]); byte j of `w` holds code_2j in its high nibble and code_2j+1 in its low one;
 * scale: fp16 [n / block].  dst: fp16 [n].  The fp16 projection entry points then run on the copy, which is how this
 * device serves NF4 weights (the packed form stays the resident one; the copy is a per-call scratch). */
int jg_dequant_nf4_f16(jg_dev* dev, uint64_t dst, uint64_t w, uint64_t scale, int64_t n, int32_t block);

/* ---- Seeded synthetic tensors (stand-in for Tensor.randn/uniform, jsgrad/tensor.ts:796-843, which the
 *      workloads replace by fixed distributions).  Counter-based, so any sub-range can be generated. */
int jg_fill_normal_f16(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t first, uint64_t n, float std);
int jg_fill_uniform_i8(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t first, uint64_t n);
int jg_fill_scale_f16(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t first, uint64_t n, float base);
int jg_fill_const_f16(jg_dev* dev, uint64_t dst, uint64_t n, float value);
/* [rows][cols] window at (row0, col0) of a [*][full_cols] tensor: a shard gets the values the whole tensor would. */
int jg_fill_normal_f16_2d(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t rows, uint64_t cols, uint64_t full_cols,
                          uint64_t row0, uint64_t col0, float std);
int jg_fill_uniform_i8_2d(jg_dev* dev, uint64_t dst, uint64_t seed, uint64_t rows, uint64_t cols, uint64_t full_cols,
                          uint64_t row0, uint64_t col0);

#ifdef __cplusplus
}
#endif
#endif /* JSGRAD_CUDA_H */
