// jsgrad/models/llama_cuda.ts — the Llama transformer of models/llama.ts on the `CUDA` device (runtime/ops_cuda.ts):
// the same class names, constructor arguments, state-dict names and call semantics, with every block step mapped onto
// the hand-written kernels of libjsgrad_cuda.so instead of a lazy graph.
//
// How it plugs in.  models/llama.ts builds `new Transformer(dim, hidden_dim, n_heads, n_layers, norm_eps, vocab_size,
// linear, embedding, n_kv_heads, rope_theta, max_context, jit, feed_forward)` and Llama3 injects Int8Linear /
// Int8Embedding through `linear` / `embedding` (models/llama3.ts:190-200).  `CudaTransformer` takes the same arguments;
// Llama3 constructs it instead of `Transformer` when the device is CUDA:
//     const T = this.device.toString().startsWith('CUDA') ? CudaTransformer : Transformer
//     this.model = new T(params.dim, params.hidden_dim, ..., this.linear === Int8Linear ? CudaInt8Linear : CudaLinear, ...)
// Weights are ordinary realized Tensors under the reference's names (`layers.3.attention.wq.weight`, ...), so
// get_state_dict / load_state_dict / Int8Linear.quantize keep working; wq | wk | wv of a layer are row windows of one
// allocation (the reference's WQKV option, models/llama.ts:63-66).
//
// Every kernel call below is a line `cu(dev, '<entry point>', <arguments in header order>)`.  The sequences are the ones
// denograd_b200/llama.py issues (the Python twin that the test-suite runs on a B200); tests/test_ts_seam.py checks
// both against ts/call_plan.json, line by line.  No Deno runtime exists where this is built, so this file has been
// type-checked by reading only.
import { Tensor } from '../tensor.ts'
import { dtypes } from '../dtype.ts'
import { Device } from '../device.ts'
import { type CUDA, CUDAGraph, cu, cu_h, check } from '../runtime/ops_cuda.ts'

/** Device address of a realized tensor (the allocator's opaque Buf is the address itself). */
const ptr_of = (t: Tensor): bigint => (t.lazydata.base.realized!._buf as bigint) + BigInt(t.lazydata.base.realized!.offset ?? 0)
const empty = (shape: number[], dtype = dtypes.half, device: string) => Tensor.empty(shape, { dtype, device }).contiguous().realize()

/** A realized device tensor with its address cached: what `cu` accepts. */
class Dev {
  ptr: bigint
  constructor(public t: Tensor) {
    this.ptr = ptr_of(t)
  }
}

export class CudaLinear {
  weight: Tensor
  scale_ptr = 0n
  constructor(public in_features: number, public out_features: number, bias = false, weight?: Tensor) {
    if (bias !== false) throw new Error('Linear bias is not used on the Llama path')
    this.weight = weight ?? Tensor.empty([out_features, in_features], { dtype: dtypes.half })
  }
  get ptr() {
    return ptr_of(this.weight)
  }
}

export class CudaInt8Linear extends CudaLinear {
  scale: Tensor
  constructor(in_features: number, out_features: number, bias = false, weight?: Tensor, scale?: Tensor) {
    super(in_features, out_features, bias, weight ?? Tensor.ones([out_features, in_features], { dtype: dtypes.int8 }))
    this.scale = scale ?? Tensor.ones([out_features], { dtype: dtypes.half })
  }
  override get scale_ptr() {
    return ptr_of(this.scale)
  }
}

export class CudaRMSNorm {
  weight: Tensor
  constructor(dim: number, public eps = 1e-6) {
    this.weight = Tensor.ones([dim], { dtype: dtypes.half })
  }
  get ptr() {
    return ptr_of(this.weight)
  }
}

export class CudaEmbedding {
  weight: Tensor
  scale_ptr = 0n
  constructor(public vocab_size: number, public embed_size: number) {
    this.weight = Tensor.empty([vocab_size, embed_size], { dtype: dtypes.half })
  }
  get ptr() {
    return ptr_of(this.weight)
  }
}

/** Activation buffers of one step for a fixed row count (what the memory planner would assign, engine/memory.ts). */
class Workspace {
  tokens: Dev; pos: Dev; seq: Dev; h: Dev; xn: Dev; qkv: Dev; attn: Dev; ffn: Dev; logits: Dev; key: Dev; next_tokens: Dev
  constructor(public B: number, dim: number, qkv_dim: number, q_dim: number, hidden: number, vocab: number, device: string) {
    const i32 = dtypes.int32
    this.tokens = new Dev(Tensor.zeros([B], { dtype: i32, device }).contiguous().realize())
    this.pos = new Dev(Tensor.zeros([B], { dtype: i32, device }).contiguous().realize())
    this.seq = new Dev(Tensor.zeros([B], { dtype: i32, device }).contiguous().realize())
    this.h = new Dev(empty([B, dim], dtypes.half, device))
    this.xn = new Dev(empty([B, dim], dtypes.half, device))
    this.qkv = new Dev(empty([B, qkv_dim], dtypes.half, device))
    this.attn = new Dev(empty([B, q_dim], dtypes.half, device))
    this.ffn = new Dev(empty([B, hidden], dtypes.half, device))
    this.logits = new Dev(empty([B, Math.max(vocab, 1)], dtypes.half, device))
    this.key = new Dev(Tensor.zeros([B], { dtype: dtypes.uint64, device }).contiguous().realize())
    this.next_tokens = new Dev(Tensor.zeros([B], { dtype: i32, device }).contiguous().realize())
  }
}

/** The model's paged K/V pool (Attention.cache_kv per layer in the reference, models/llama.ts:78-90). */
class KVCache {
  handle: Deno.PointerValue = null
  fused_attention = true
  constructor(dev: CUDA, n_layers: number, n_heads: number, n_kv_heads: number, head_dim: number, max_context: number, max_batch: number, page_size = 64) {
    const pages_per_seq = Math.ceil(max_context / page_size)
    const desc = new Int32Array([n_layers, n_kv_heads, head_dim, page_size, pages_per_seq * max_batch, max_batch, pages_per_seq, n_heads, 0])
    const out = new BigUint64Array(1)
    cu(dev, 'jg_kvcache_create', desc as unknown as bigint, out as unknown as bigint)
    this.handle = Deno.UnsafePointer.create(out[0])
  }
}

export class CudaAttention {
  n_kv_heads: number
  head_dim: number
  n_rep: number
  wqkv: CudaLinear
  wq: CudaLinear
  wk: CudaLinear
  wv: CudaLinear
  wo: CudaLinear
  layer = 0
  constructor(dim: number, public n_heads: number, n_kv_heads: number | undefined, public max_context: number, linear: typeof CudaLinear = CudaLinear) {
    this.n_kv_heads = n_kv_heads !== undefined ? n_kv_heads : n_heads
    this.head_dim = Math.trunc(dim / n_heads)
    this.n_rep = Math.trunc(this.n_heads / this.n_kv_heads)
    const q_out = this.n_heads * this.head_dim, kv_out = this.n_kv_heads * this.head_dim
    this.wqkv = new linear(dim, q_out + 2 * kv_out, false)
    const rows = (a: number, b: number) => this.wqkv.weight.shrink([[a, b], undefined])
    this.wq = new linear(dim, q_out, false, rows(0, q_out))
    this.wk = new linear(dim, kv_out, false, rows(q_out, q_out + kv_out))
    this.wv = new linear(dim, kv_out, false, rows(q_out + kv_out, q_out + 2 * kv_out))
    this.wo = new linear(q_out, dim, false)
  }
}

export class CudaFeedForward {
  w1: CudaLinear
  w2: CudaLinear
  w3: CudaLinear
  constructor(dim: number, hidden_dim: number, linear: typeof CudaLinear = CudaLinear) {
    this.w1 = new linear(dim, hidden_dim, false)
    this.w2 = new linear(hidden_dim, dim, false)
    this.w3 = new linear(dim, hidden_dim, false) // the gate in Gated Linear Unit
  }
}

/** Whether RMSNorm runs as its own kernel ahead of a projection.  The matrix-vector kernels fold the norm into their
 *  prologue; the tensor-core kernels take normalised rows: fp16 weights from 3 rows on; int8 weights beyond one row, or
 *  when a row of `dim` halves does not fit the shared memory of the int8 matrix-vector kernel (dim a multiple of 512). */
export const norm_first = (rows: number, int8: boolean, dim: number): boolean => {
  if (!int8) return rows >= 3
  return rows > 1 || dim <= 0 || dim % 512 !== 0 || 2 * (rows * (2 * dim + 16) + 4096) > 228 * 1024
}

export class CudaTransformerBlock {
  attention: CudaAttention
  feed_forward: CudaFeedForward
  attention_norm: CudaRMSNorm
  ffn_norm: CudaRMSNorm
  constructor(dim: number, hidden_dim: number, n_heads: number, n_kv_heads: number | undefined, norm_eps: number, max_context: number, linear: typeof CudaLinear = CudaLinear, feed_forward: typeof CudaFeedForward = CudaFeedForward) {
    this.attention = new CudaAttention(dim, n_heads, n_kv_heads, max_context, linear)
    this.feed_forward = new feed_forward(dim, hidden_dim, linear)
    this.attention_norm = new CudaRMSNorm(dim, norm_eps)
    this.ffn_norm = new CudaRMSNorm(dim, norm_eps)
  }

  /** h = x + attention(attention_norm(x)); h + feed_forward(ffn_norm(h))  (models/llama.ts:124-127), one token per
   *  row, the row counts norm_first() lets through: norms folded into the projections' prologues,
   *  residual adds and SiLU * up into their epilogues, RoPE + cache write + attention in one cluster launch. */
  decode_step_fused = (dev: CUDA, ws: Workspace, kv: KVCache, freqs_cis: Dev, freqs_rows: number, dim: number) => {
    const a = this.attention, f = this.feed_forward, B = ws.B
    cu(dev, 'jg_norm_linear', ws.qkv, ws.h, this.attention_norm, this.attention_norm.eps, a.wqkv, a.wqkv.scale_ptr, B, a.wqkv.out_features, dim)
    cu(dev, 'jg_attn_decode_fused', kv.handle, a.layer, ws.attn, ws.qkv, freqs_cis, freqs_rows, ws.pos, B, a.n_heads)
    cu(dev, 'jg_linear', ws.h, ws.attn, a.wo, a.wo.scale_ptr, ws.h, B, a.wo.out_features, a.wo.in_features)
    cu(dev, 'jg_norm_swiglu', ws.ffn, ws.h, this.ffn_norm, this.ffn_norm.eps, f.w1, f.w1.scale_ptr, f.w3, f.w3.scale_ptr, B, f.w1.out_features, dim)
    cu(dev, 'jg_linear', ws.h, ws.ffn, f.w2, f.w2.scale_ptr, ws.h, B, f.w2.out_features, f.w2.in_features)
  }

  /** The same block for more rows per step: the norms run as their own kernel and the projections take normalised
   *  rows (tensor-core kernels). */
  decode_step_rows = (dev: CUDA, ws: Workspace, kv: KVCache, freqs_cis: Dev, freqs_rows: number, dim: number) => {
    const a = this.attention, f = this.feed_forward, B = ws.B
    cu(dev, 'jg_rmsnorm', ws.xn, ws.h, this.attention_norm, B, dim, this.attention_norm.eps)
    cu(dev, 'jg_linear', ws.qkv, ws.xn, a.wqkv, a.wqkv.scale_ptr, 0, B, a.wqkv.out_features, dim)
    cu(dev, 'jg_attn_decode_fused', kv.handle, a.layer, ws.attn, ws.qkv, freqs_cis, freqs_rows, ws.pos, B, a.n_heads)
    cu(dev, 'jg_linear', ws.h, ws.attn, a.wo, a.wo.scale_ptr, ws.h, B, a.wo.out_features, a.wo.in_features)
    cu(dev, 'jg_rmsnorm', ws.xn, ws.h, this.ffn_norm, B, dim, this.ffn_norm.eps)
    cu(dev, 'jg_norm_swiglu', ws.ffn, ws.xn, 0, this.ffn_norm.eps, f.w1, f.w1.scale_ptr, f.w3, f.w3.scale_ptr, B, f.w1.out_features, dim)
    cu(dev, 'jg_linear', ws.h, ws.ffn, f.w2, f.w2.scale_ptr, ws.h, B, f.w2.out_features, f.w2.in_features)
  }

  /** One chunk of a multi-position call (seqlen > 1, models/llama.ts:201-213): R = batch * positions rows,
   *  position-major; every row attends to the cache up to its own position, which is what the reference's additive
   *  causal mask (:208) computes. */
  prefill_chunk = (dev: CUDA, ws: Workspace, kv: KVCache, freqs_cis: Dev, freqs_rows: number, dim: number, batch: number, positions: number) => {
    const a = this.attention, f = this.feed_forward, R = ws.B
    cu(dev, 'jg_rmsnorm', ws.xn, ws.h, this.attention_norm, R, dim, this.attention_norm.eps)
    cu(dev, 'jg_linear', ws.qkv, ws.xn, a.wqkv, a.wqkv.scale_ptr, 0, R, a.wqkv.out_features, dim)
    cu(dev, 'jg_rope_kvwrite_rows', kv.handle, a.layer, ws.qkv, freqs_cis, freqs_rows, ws.pos, ws.seq, R, a.n_heads)
    cu(dev, 'jg_attn_chunk', kv.handle, a.layer, ws.attn, ws.qkv, ws.pos, ws.seq, batch, positions, a.n_heads)
    cu(dev, 'jg_linear', ws.h, ws.attn, a.wo, a.wo.scale_ptr, ws.h, R, a.wo.out_features, a.wo.in_features)
    cu(dev, 'jg_rmsnorm', ws.xn, ws.h, this.ffn_norm, R, dim, this.ffn_norm.eps)
    cu(dev, 'jg_norm_swiglu', ws.ffn, ws.xn, 0, this.ffn_norm.eps, f.w1, f.w1.scale_ptr, f.w3, f.w3.scale_ptr, R, f.w1.out_features, dim)
    cu(dev, 'jg_linear', ws.h, ws.ffn, f.w2, f.w2.scale_ptr, ws.h, R, f.w2.out_features, f.w2.in_features)
  }
}

/** The model's decode step as one persistent kernel (jg_step_create): the table of the layers' tensors and the kernel's
 *  scratch.  The tensors' addresses are fixed at creation, like those a captured graph holds.  `handle` stays null when
 *  the library has no such kernel for the model's shape (status 95): the launch-per-op step is used then. */
class StepPlan {
  handle: Deno.PointerValue = null
  private table: BigUint64Array // kept alive: the library reads it during create only, but the desc points at it
  constructor(dev: CUDA, m: CudaTransformer) {
    this.table = new BigUint64Array(m.layers.length * 7)
    m.layers.forEach((l, i) => this.table.set([l.attention_norm.ptr, l.attention.wqkv.ptr, l.attention.wo.ptr, l.ffn_norm.ptr, l.feed_forward.w1.ptr, l.feed_forward.w3.ptr, l.feed_forward.w2.ptr], i * 7))
    const desc = new DataView(new ArrayBuffer(88)) // jg_step_desc: 6 x int32, float, int32, 6 x uint64, int64
    ;[m.layers.length, m.dim, m.hidden_dim, m.n_heads, m.vocab_size, m.max_context * 2].forEach((v, i) => desc.setInt32(4 * i, v, true))
    desc.setFloat32(24, m.norm.eps, true)
    desc.setInt32(28, 0, true) // vocab_offset: one device holds the whole vocabulary
    const table_addr = BigInt(Deno.UnsafePointer.value(Deno.UnsafePointer.of(this.table)))
    // the last two: no communicator (one device), embedding rows = vocabulary
    ;[table_addr, m.tok_embeddings.ptr, m.norm.ptr, m.output.ptr, m.freqs_cis.ptr, 0n].forEach((v, i) => desc.setBigUint64(32 + 8 * i, v, true))
    desc.setBigInt64(80, BigInt(m.vocab_size), true)
    const out = new BigUint64Array(1)
    try {
      cu_h('jg_step_create', dev.handle, m.kv.handle as unknown as bigint, new Uint8Array(desc.buffer) as unknown as bigint, out as unknown as bigint)
      this.handle = Deno.UnsafePointer.create(out[0])
    } catch (e) {
      if (!String(e).includes('status 95')) throw e
    }
  }
}

export class CudaTransformer {
  layers: CudaTransformerBlock[]
  norm: CudaRMSNorm
  tok_embeddings: CudaEmbedding
  output: CudaLinear
  freqs_cis!: Dev
  head_dim: number
  dev!: CUDA
  kv!: KVCache
  private step_plan?: StepPlan
  private ws = new Map<number, Workspace>()
  private step_graph = new Map<number, CUDAGraph>()
  private calls = new Map<number, number>()
  constructor(public dim: number, public hidden_dim: number, public n_heads: number, n_layers: number, norm_eps: number, public vocab_size: number, linear: typeof CudaLinear = CudaLinear, embedding: typeof CudaEmbedding = CudaEmbedding, public n_kv_heads?: number, public rope_theta = 10000, public max_context = 1024, public jit = true, feed_forward: typeof CudaFeedForward = CudaFeedForward, public max_batch = 1) {
    this.head_dim = Math.trunc(dim / n_heads)
    this.layers = Array.from({ length: n_layers }, () => new CudaTransformerBlock(dim, hidden_dim, n_heads, n_kv_heads, norm_eps, max_context, linear, feed_forward))
    this.layers.forEach((l, i) => l.attention.layer = i)
    this.norm = new CudaRMSNorm(dim, norm_eps)
    this.tok_embeddings = new embedding(vocab_size, dim)
    this.output = embedding === CudaEmbedding ? new CudaLinear(dim, vocab_size, false) : new linear(dim, vocab_size, false)
  }

  /** Realize the weights on the device, build the RoPE table (precompute_freqs_cis cast to fp16, models/llama.ts:10-14,
   *  205) and the K/V pool.  Awaited once, after load_state_dict. */
  init = async (device = Device.DEFAULT) => {
    this.dev = Device.get(device) as unknown as CUDA
    await this.dev.init()
    const table = empty([this.max_context * 2, this.head_dim / 2, 2], dtypes.half, device)
    this.freqs_cis = new Dev(table)
    cu(this.dev, 'jg_freqs_cis', this.freqs_cis, this.head_dim, this.max_context * 2, this.rope_theta)
    this.kv = new KVCache(this.dev, this.layers.length, this.n_heads, this.n_kv_heads ?? this.n_heads, this.head_dim, this.max_context, this.max_batch)
  }

  private workspace = (B: number, logits = true) => {
    const key = logits ? B : -B
    if (!this.ws.has(key)) {
      const kvh = this.n_kv_heads ?? this.n_heads
      this.ws.set(key, new Workspace(B, this.dim, (this.n_heads + 2 * kvh) * this.head_dim, this.n_heads * this.head_dim, this.hidden_dim, logits ? this.vocab_size : 0, this.dev.device))
    }
    return this.ws.get(key)!
  }

  /** The plan of the single-kernel step when this model and row count can take it: fp16 weights, 1-2 rows. */
  private single_kernel_step = (B: number): StepPlan | undefined => {
    if (B > 2 || this.output.scale_ptr !== 0n || this.tok_embeddings.scale_ptr !== 0n) return undefined
    if (this.step_plan === undefined) this.step_plan = new StepPlan(this.dev, this)
    return this.step_plan.handle !== null ? this.step_plan : undefined
  }

  /** The whole step as one launch of the persistent kernel (one step, nothing fed back). */
  private decode_step_single = (plan: StepPlan, ws: Workspace, B: number) => {
    cu_h('jg_step_run', plan.handle, ws.tokens, ws.pos, ws.h, ws.qkv, ws.attn, ws.ffn, ws.logits, ws.next_tokens, B, 1, 0)
  }

  /** One token per row: reads ws.tokens / ws.pos, leaves the fp16 logits and the greedy ids in the workspace. */
  private decode_step = (ws: Workspace) => {
    const dev = this.dev, B = ws.B, int8 = this.output.scale_ptr !== 0n
    const plan = this.single_kernel_step(B)
    if (plan !== undefined) return this.decode_step_single(plan, ws, B)
    const fused = !norm_first(B, int8, this.dim)
    cu(dev, 'jg_embed', ws.h, ws.tokens, this.tok_embeddings, this.tok_embeddings.scale_ptr, B, this.dim, this.vocab_size)
    for (const layer of this.layers) {
      if (fused) layer.decode_step_fused(dev, ws, this.kv, this.freqs_cis, this.max_context * 2, this.dim)
      else layer.decode_step_rows(dev, ws, this.kv, this.freqs_cis, this.max_context * 2, this.dim)
    }
    if (fused) {
      cu(dev, 'jg_norm_logits_argmax_shard', ws.logits, ws.key, ws.h, this.norm, this.norm.eps, this.output, this.output.scale_ptr, B, this.vocab_size, this.dim, 0)
    } else {
      cu(dev, 'jg_rmsnorm', ws.xn, ws.h, this.norm, B, this.dim, this.norm.eps)
      cu(dev, 'jg_norm_logits_argmax_shard', ws.logits, ws.key, ws.xn, 0, this.norm.eps, this.output, this.output.scale_ptr, B, this.vocab_size, this.dim, 0)
    }
    cu(dev, 'jg_argmax_finalize', ws.next_tokens, ws.key, B)
  }

  /** The token of the step: the greedy pick already made, or `sample` over the step's logits (models/llama.ts:131-185)
   *  with one uniform sample per row from Tensor.rand. */
  private pick = async (ws: Workspace, temperature: number, top_k: number, top_p: number, alpha_f: number, alpha_p: number) => {
    if (temperature >= 1e-6) {
      const u = new Dev(await Tensor.rand([ws.B], undefined, { device: this.dev.device }).realize())
      cu(this.dev, 'jg_sample', ws.next_tokens, ws.logits, u, 0, ws.B, this.vocab_size, temperature, top_k, top_p, alpha_f, alpha_p)
    }
    return ws.next_tokens.t
  }

  forward = async (tokens: Tensor, start_pos: number, temperature: number, top_k: number, top_p: number, alpha_f: number, alpha_p: number) => {
    const [bsz, seqlen] = tokens.shape_num
    const toks = (await tokens.tolist()) as number[][]
    const wsb = this.workspace(bsz)
    if (seqlen === 1) {
      await wsb.tokens.t.assign(new Tensor(toks.map((r) => r[0]), { dtype: dtypes.int32, device: this.dev.device })).realize()
      await wsb.pos.t.assign(Tensor.full([bsz], start_pos, { dtype: dtypes.int32, device: this.dev.device })).realize()
      this.decode_step(wsb)
      return await this.pick(wsb, temperature, top_k, top_p, alpha_f, alpha_p)
    }
    // several positions: chunks of up to 2048 rows, position-major (row = s * bsz + b)
    const per = Math.max(1, Math.trunc(2048 / bsz))
    for (let s0 = 0; s0 < seqlen; s0 += per) {
      const sc = Math.min(per, seqlen - s0), R = bsz * sc, ws = this.workspace(R, false), dev = this.dev
      const flat: number[] = [], pos: number[] = [], seq: number[] = []
      for (let s = 0; s < sc; s++) for (let b = 0; b < bsz; b++) flat.push(toks[b][s0 + s]), pos.push(start_pos + s0 + s), seq.push(b)
      await ws.tokens.t.assign(new Tensor(flat, { dtype: dtypes.int32, device: dev.device })).realize()
      await ws.pos.t.assign(new Tensor(pos, { dtype: dtypes.int32, device: dev.device })).realize()
      await ws.seq.t.assign(new Tensor(seq, { dtype: dtypes.int32, device: dev.device })).realize()
      cu(dev, 'jg_embed', ws.h, ws.tokens, this.tok_embeddings, this.tok_embeddings.scale_ptr, R, this.dim, this.vocab_size)
      for (const layer of this.layers) layer.prefill_chunk(dev, ws, this.kv, this.freqs_cis, this.max_context * 2, this.dim, bsz, sc)
      if (s0 + per >= seqlen) { // the rows of the last position meet the output layer (the reference keeps logits[:, -1, :], :210)
        const h_last = ws.h.ptr + BigInt(2 * this.dim * (R - bsz)), xn_last = ws.xn.ptr + BigInt(2 * this.dim * (R - bsz))
        cu(dev, 'jg_rmsnorm', xn_last, h_last, this.norm, bsz, this.dim, this.norm.eps)
        cu(dev, 'jg_norm_logits_argmax_shard', wsb.logits, wsb.key, xn_last, 0, this.norm.eps, this.output, this.output.scale_ptr, bsz, this.vocab_size, this.dim, 0)
        cu(dev, 'jg_argmax_finalize', wsb.next_tokens, wsb.key, bsz)
      }
    }
    return await this.pick(wsb, temperature, top_k, top_p, alpha_f, alpha_p)
  }

  /** Transformer.call (models/llama.ts:214-220): single-token calls after position 0 replay a captured step, the role
   *  TinyJit has in the reference (call 0 eager, call 1 captured, later calls replayed: engine/jit.ts:273-353). */
  call = async (tokens: Tensor, start_pos: number, temperature = 0.0, top_k = 0, top_p = 0.8, alpha_f = 0.0, alpha_p = 0.0) => {
    const [bsz, seqlen] = tokens.shape_num
    if (seqlen === 1 && this.jit && start_pos !== 0) {
      const ws = this.workspace(bsz), n = this.calls.get(bsz) ?? 0
      await ws.tokens.t.assign(tokens.reshape([bsz]).cast(dtypes.int32)).realize()
      await ws.pos.t.assign(Tensor.full([bsz], start_pos, { dtype: dtypes.int32, device: this.dev.device })).realize()
      if (n === 0) this.decode_step(ws)
      else {
        if (n === 1) this.step_graph.set(bsz, await CUDAGraph.capture(this.dev, [], [], new Map(), async () => this.decode_step(ws)))
        this.step_graph.get(bsz)!.call([], new Map())
      }
      this.calls.set(bsz, n + 1)
      return await this.pick(ws, temperature, top_k, top_p, alpha_f, alpha_p)
    }
    return await this.forward(tokens, start_pos, temperature, top_k, top_p, alpha_f, alpha_p)
  }
}
export { check, cu_h }
