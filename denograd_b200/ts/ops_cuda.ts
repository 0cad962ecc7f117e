// jsgrad/runtime/ops_cuda.ts — the `CUDA` device for jsgrad, backed by libjsgrad_cuda.so (hand-written sm_100a
// kernels behind a C ABI, see include/jsgrad_cuda.h).
//
// Drop this file into jsgrad/runtime/ and register it in jsgrad/env/deno.ts:
//     import { CUDA } from '../runtime/ops_cuda.ts'
//     override DEVICES = { CLANG, WEBGPU: DAWN, WGPU: WEBGPU, WASM, JS, DISK, CLOUD, CUDA }
//
// It follows the shape of the reference's own devices: ops_clang.ts (Program bound through env.dlopen with
// 'pointer' / 'i32' parameters) and ops_dawn.ts (library opened once in init(), opaque native buffers).  The engine
// above it is unchanged: Tensor, nn.Linear, models/llama keep their API.  No Deno runtime exists where this package
// is built and tested, so this file is kept mechanically identical to denograd_b200/ffi.py + device.py, which make
// the same C calls and are what the test-suite drives.
import { Allocator, type BufferSpec, Compiled, Compiler, Program, type ProgramCallArgs } from './allocator.ts'
import type { MemoryView } from '../helpers/memoryview.ts'
import { env } from '../env/index.ts'
import { vars } from '../helpers/helpers.ts'
import { CUDARenderer } from '../renderer/cstyle.ts'
import type { Buffer } from '../device.ts'
import { type ExecItem } from '../engine/realize.ts'
import { GraphRunner } from '../engine/jit.ts'
import type { Variable } from '../ops.ts'

const u64 = 'u64', i32 = 'i32', f32 = 'f32', f64 = 'f64', ptr = 'pointer', buf = 'buffer', usize = 'usize'
const fn = (parameters: readonly string[], nonblocking = false) => ({ parameters, result: 'i32', nonblocking } as const)

// One entry per function of include/jsgrad_cuda.h (same order, same types).
export const SYMBOLS = {
  jg_device_count: fn([buf]),
  jg_device_open: fn([i32, buf]),
  jg_device_close: fn([ptr]),
  jg_device_sync: fn([ptr], true),
  jg_device_props: fn([ptr, buf]),
  jg_last_error: { parameters: [], result: 'pointer' },
  jg_launch_count: fn([ptr, buf]),
  jg_alloc: fn([ptr, usize, buf]),
  jg_free: fn([ptr, u64]),
  jg_copyin: fn([ptr, u64, buf, usize]),
  jg_copyout: fn([ptr, buf, u64, usize], true),
  jg_transfer: fn([ptr, u64, ptr, u64, usize]),
  jg_memset: fn([ptr, u64, i32, usize]),
  jg_copy: fn([ptr, u64, u64, usize]),
  jg_host_alloc: fn([usize, buf]),
  jg_host_free: fn([ptr]),
  jg_copyin_async: fn([ptr, u64, ptr, usize]),
  jg_copyout_async: fn([ptr, ptr, u64, usize]),
  jg_timer_start: fn([ptr]),
  jg_timer_stop: fn([ptr, buf], true),
  jg_cuda_compile: fn([buf, buf, buf, buf]),
  jg_cuda_image_free: fn([ptr]),
  jg_program_load: fn([ptr, buf, buf, u64, buf]),
  jg_program_call: fn([ptr, buf, i32, buf, i32, buf, buf]),
  jg_program_destroy: fn([ptr]),
  jg_graph_begin: fn([ptr]),
  jg_graph_end: fn([ptr, buf]),
  jg_graph_launch: fn([ptr, ptr]),
  jg_graph_destroy: fn([ptr]),
  jg_embed: fn([ptr, u64, u64, u64, u64, i32, i32, i32]),
  jg_rmsnorm: fn([ptr, u64, u64, u64, i32, i32, f32]),
  jg_linear: fn([ptr, u64, u64, u64, u64, u64, i32, i32, i32]),
  jg_norm_linear: fn([ptr, u64, u64, u64, f32, u64, u64, i32, i32, i32]),
  jg_norm_swiglu: fn([ptr, u64, u64, u64, f32, u64, u64, u64, u64, i32, i32, i32]),
  jg_swiglu: fn([ptr, u64, u64, u64, 'i64']),
  jg_norm_logits_argmax: fn([ptr, u64, u64, u64, u64, f32, u64, u64, i32, i32, i32]),
  jg_argmax_finalize: fn([ptr, u64, u64, i32]),
  jg_argmax: fn([ptr, u64, u64, i32, i32]),
  jg_sample: fn([ptr, u64, u64, u64, u64, i32, i32, f32, i32, f32, f32, f32]),
  jg_freqs_cis: fn([ptr, u64, i32, i32, f64]),
  jg_kvcache_create: fn([ptr, buf, buf]),
  jg_kvcache_destroy: fn([ptr]),
  jg_kvcache_set_block_table: fn([ptr, buf]),
  jg_kvcache_bytes: fn([ptr, buf]),
  jg_rope_kvwrite: fn([ptr, ptr, i32, u64, u64, i32, u64, i32, i32]),
  jg_attn_decode: fn([ptr, ptr, i32, u64, u64, u64, i32, i32]),
  jg_attn_decode_fused: fn([ptr, ptr, i32, u64, u64, u64, i32, u64, i32, i32]),
  jg_rope_kvwrite_rows: fn([ptr, ptr, i32, u64, u64, i32, u64, u64, i32, i32]),
  jg_attn_rows: fn([ptr, ptr, i32, u64, u64, u64, u64, i32, i32]),
  jg_attn_chunk: fn([ptr, ptr, i32, u64, u64, u64, u64, i32, i32, i32]),
  jg_attn_decode_noalloc: fn([ptr, u64, u64, u64, u64, u64, u64, i32, i32, i32, i32, i32, i32, i32, i32]),
  jg_pos_advance: fn([ptr, u64, i32]),
  jg_dequant_i8_f16: fn([ptr, u64, u64, u64, 'i64', 'i64']),
  jg_dequant_nf4_f16: fn([ptr, u64, u64, u64, 'i64', i32]),
  jg_step_create: fn([ptr, ptr, buf, buf]),
  jg_step_destroy: fn([ptr]),
  jg_step_run: fn([ptr, u64, u64, u64, u64, u64, u64, u64, u64, i32, i32, i32]),
  jg_fill_normal_f16: fn([ptr, u64, u64, u64, u64, f32]),
  jg_fill_uniform_i8: fn([ptr, u64, u64, u64, u64]),
  jg_fill_scale_f16: fn([ptr, u64, u64, u64, u64, f32]),
  jg_fill_const_f16: fn([ptr, u64, u64, f32]),
  jg_fill_normal_f16_2d: fn([ptr, u64, u64, u64, u64, u64, u64, u64, f32]),
  jg_fill_uniform_i8_2d: fn([ptr, u64, u64, u64, u64, u64, u64, u64]),
  jg_comm_unique_id: fn([buf, buf]),
  jg_comm_init: fn([ptr, buf, buf, i32, i32, buf]),
  jg_comm_destroy: fn([ptr]),
  jg_allreduce_sum_f32: fn([ptr, u64, u64]),
  jg_allreduce_max_u64: fn([ptr, u64, u64]),
  jg_comm_peer_export: fn([ptr, ptr]),
  jg_comm_peer_open: fn([ptr, ptr]),
  jg_comm_peer_capacity: fn([ptr, ptr]),
  jg_peer_allreduce_residual: fn([ptr, u64, u64, u64]),
  jg_peer_allreduce_max_u64: fn([ptr, u64, u64]),
  jg_linear_allreduce_residual: fn([ptr, u64, u64, u64, u64, i32, i32, i32]),
  jg_tp_linear_push: fn([ptr, u64, u64, u64, i32, i32, i32]),
  jg_tp_norm_linear: fn([ptr, u64, u64, u64, u64, f32, u64, u64, i32, i32, i32]),
  jg_tp_norm_swiglu: fn([ptr, u64, u64, u64, u64, f32, u64, u64, u64, u64, i32, i32, i32]),
  jg_tp_norm_logits_argmax: fn([ptr, u64, u64, u64, u64, u64, f32, u64, u64, i32, i32, i32, i32]),
  jg_comm_peer_partial: fn([ptr, buf, buf]),
  jg_peer_allreduce2_residual: fn([ptr, u64, u64]),
  jg_comm_init_all: fn([i32, buf, buf, buf]),
  jg_comm_group_begin: fn([]),
  jg_comm_group_end: fn([]),
  jg_linear_partial: fn([ptr, u64, u64, u64, u64, i32, i32, i32]),
  jg_residual_add_f32: fn([ptr, u64, u64, 'i64']),
  jg_norm_logits_argmax_shard: fn([ptr, u64, u64, u64, u64, f32, u64, u64, i32, i32, i32, i32]),
} as const

type Lib = { symbols: Record<keyof typeof SYMBOLS, (...a: any[]) => any> }
let lib: Lib | undefined

export const check = (status: number) => {
  if (status !== 0) throw new Error(`[jsgrad_cuda status ${status}] ${env.getCString(lib!.symbols.jg_last_error())}`)
}
const out64 = () => new BigUint64Array(1)

/** One kernel entry point on one device: `cu(dev, 'jg_linear', y, x, ...)`.  Arguments may be device addresses
 *  (bigint), numbers, or anything with a `.ptr` (the layers' tensors): the address is taken here, so the call sites read
 *  like the argument lists of include/jsgrad_cuda.h.  The first C argument (the device handle) is supplied here. */
export const cu = (dev: CUDA, entry: keyof typeof SYMBOLS, ...args: (bigint | number | { ptr: bigint } | undefined)[]) =>
  check(lib!.symbols[entry](dev.handle, ...args.map((a) => a === undefined ? 0n : (typeof a === 'object' ? a.ptr : a))))
/** The same for entry points whose first argument is another handle (a kv cache, a communicator). */
export const cu_h = (entry: keyof typeof SYMBOLS, handle: Deno.PointerValue, ...args: (bigint | number | { ptr: bigint } | undefined)[]) =>
  check(lib!.symbols[entry](handle, ...args.map((a) => a === undefined ? 0n : (typeof a === 'object' ? a.ptr : a))))

/** Buf = device address (bigint).  Allocator contract: jsgrad/runtime/allocator.ts:28-47. */
export class CUDAAllocator extends Allocator<bigint> {
  constructor(public dev: CUDA) { // BufferXfer reads `allocator.dev` on both sides (engine/realize.ts:126)
    super()
  }
  _alloc = (size: number, _options: BufferSpec) => {
    const o = out64()
    check(lib!.symbols.jg_alloc(this.dev.handle, BigInt(size), o))
    return o[0]
  }
  _free = (opaque: bigint, _options: BufferSpec) => check(lib!.symbols.jg_free(this.dev.handle, opaque))
  _copyin = (dest: bigint, src: MemoryView) => check(lib!.symbols.jg_copyin(this.dev.handle, dest, src.bytes, BigInt(src.byteLength)))
  _copyout = async (dest: MemoryView, src: bigint) => check(await lib!.symbols.jg_copyout(this.dev.handle, dest.bytes, src, BigInt(dest.byteLength)))
  override _offset = (buf: bigint, _size: number, offset: number) => buf + BigInt(offset)
  override _transfer = (dest: bigint, src: bigint, sz: number, src_dev: CUDA, dest_dev: CUDA) =>
    check(lib!.symbols.jg_transfer(dest_dev.handle, dest, src_dev.handle, src, BigInt(sz)))
}

const is_descriptor = (b: Uint8Array | string) => (typeof b === 'string' ? b.charCodeAt(0) : b[0]) === 0x7b // '{'
const cstr = (s: string) => new TextEncoder().encode(s + '\0')

/** Compiler (allocator.ts:123-139).  Two kinds of "source" reach it: the kernel descriptors the layers of
 *  llama_cuda.ts write (JSON, passed through as bytes — nothing to compile), and CUDA C from the reference's own
 *  CUDARenderer (renderer/cstyle.ts:348-419) for an AST without a hand-written kernel, which NVRTC turns into a cubin
 *  (jg_cuda_compile; a source that does not compile throws with the compiler's log, like ops_clang.ts:21). */
export class CUDACompiler extends Compiler {
  constructor(public arch = 'sm_100a') {
    super(`compile_cuda_${arch}`)
  }
  override compile = (src: string): Uint8Array => {
    if (is_descriptor(src)) return new TextEncoder().encode(src)
    const image = out64(), size = out64()
    check(lib!.symbols.jg_cuda_compile(cstr(src), cstr(this.arch), image, size))
    const p = Deno.UnsafePointer.create(image[0])
    try {
      return new Uint8Array(Deno.UnsafePointerView.getArrayBuffer(p!, Number(size[0]))).slice()
    } finally {
      check(lib!.symbols.jg_cuda_image_free(p))
    }
  }
}

/** Program contract: allocator.ts:98-107.  `lib` bytes are either a UTF-8 descriptor `{entry, order}` — a kernel of the
 *  library addressed by name: which entry point, and how its arguments interleave buffer slots (numbers), symbolic
 *  variables from args.vals ('v0', 'v1', ...) and literals — or a cubin from CUDACompiler, loaded once
 *  (jg_program_load) and launched over args.global_size x args.local_size with the buffers as pointers and
 *  args.vals as 32-bit ints (jg_program_call; argument order of ops_clang.ts:44-52).  The class is created per device
 *  (`CUDAProgram.bind(dev)`), because `Runtime.init(name, lib)` carries no device (engine/realize.ts:52-54). */
export class CUDAProgram extends Program {
  static bind = (dev: CUDA): typeof Program =>
    class extends CUDAProgram {
      static override init = (name: string, lib: Uint8Array) => new this(name, lib, dev)
    } as unknown as typeof Program
  program: Deno.PointerValue = null
  constructor(name: string, lib: Uint8Array, public dev: CUDA) {
    super(name, lib)
    if (!lib?.length) throw new Error('Lib is empty')
    if (!name) throw new Error("Name can't be undefined")
    if (!is_descriptor(lib)) {
      const o = out64()
      check(lib!.symbols.jg_program_load(dev.handle, cstr(name), lib, BigInt(lib.length), o))
      this.program = Deno.UnsafePointer.create(o[0])
    }
  }
  override call = async (bufs: bigint[], args: ProgramCallArgs, wait = false) => {
    if (wait) check(lib!.symbols.jg_timer_start(this.dev.handle))
    if (this.program) {
      const vals = args.vals ?? []
      if (vals.some((x) => x === undefined)) throw new Error(`${vals}`)
      const three = (v?: number[]) => v ? new Uint32Array([...v, 1, 1, 1].slice(0, 3)) : null
      check(lib!.symbols.jg_program_call(this.program, new BigUint64Array(bufs), bufs.length, new Int32Array(vals), vals.length, three(args.global_size), three(args.local_size)))
    } else {
      const d = JSON.parse(new TextDecoder().decode(this.lib)) as { entry: keyof typeof SYMBOLS; order: (number | string)[] }
      const argv = d.order.map((o) => typeof o === 'number' ? bufs[o] : (o.startsWith('v') ? args.vals![Number(o.slice(1))] : Number(o)))
      check(lib!.symbols[d.entry](this.dev.handle, ...argv))
    }
    if (wait) {
      const s = new Float64Array(1)
      check(await lib!.symbols.jg_timer_stop(this.dev.handle, s))
      return s[0]
    }
  }
  /** Unloads a compiled kernel's module (descriptor programs hold nothing). */
  destroy = () => {
    if (this.program) check(lib!.symbols.jg_program_destroy(this.program))
    this.program = null
  }
}

/** The device's renderer is the reference's own CUDARenderer: an AST that the scheduler hands to `render` has no
 *  hand-written kernel behind it and is generated, compiled (CUDACompiler) and launched (CUDAProgram) like on any
 *  other compiled device.  The layers of llama_cuda.ts bypass it with kernel descriptors (one per entry point they
 *  call), written by `descriptor`. */
export class CUDADescriptorRenderer extends CUDARenderer {
  constructor() {
    super('sm_100')
  }
  static descriptor = (entry: keyof typeof SYMBOLS, order: (number | string)[]) => JSON.stringify({ entry, order })
}

/** A captured kernel list replayed with one launch: the GraphRunner TinyJit asks `Compiled.graph` for
 *  (engine/jit.ts:21-29,71-141).  Varying values (tokens, start_pos) live in device memory, so `input_replace` /
 *  `var_vals_replace` have nothing to patch; `capture` records the launches of `body`, `call` replays them. */
export class CUDAGraph extends GraphRunner {
  handle: Deno.PointerValue = null
  cuda!: CUDA
  static capture = async (dev: CUDA, jit_cache: ExecItem[], input_rawbuffers: Buffer[], var_vals: Map<Variable, number>, body: () => Promise<void>) => {
    const g = new CUDAGraph(jit_cache, input_rawbuffers, var_vals)
    g.cuda = dev
    check(lib!.symbols.jg_graph_begin(dev.handle))
    try {
      await body()
    } finally {
      const o = out64()
      check(lib!.symbols.jg_graph_end(dev.handle, o))
      g.handle = Deno.UnsafePointer.create(o[0])
    }
    return g
  }
  override call = (_rawbufs: Buffer[], _var_vals: Map<Variable, number>, wait = false) => {
    if (wait) check(lib!.symbols.jg_timer_start(this.cuda.handle))
    check(lib!.symbols.jg_graph_launch(this.cuda.handle, this.handle))
    if (!wait) return undefined
    const s = new Float64Array(1)
    check(lib!.symbols.jg_timer_stop(this.cuda.handle, s))
    return s[0]
  }
  destroy = () => {
    if (this.handle) check(lib!.symbols.jg_graph_destroy(this.handle))
    this.handle = null
  }
}

export class CUDA extends Compiled {
  handle: Deno.PointerValue = null
  ordinal: number
  constructor(device: string) {
    super(device, undefined, new CUDADescriptorRenderer(), new CUDACompiler(), undefined, undefined)
    this.ordinal = device.includes(':') ? Number(device.split(':')[1]) : 0
    this.allocator = new CUDAAllocator(this)
    this.runtime = CUDAProgram.bind(this) // per device: two CUDA:n devices in one process keep their own handles
    // TinyJit batches this device's CompiledRunners through `graph` (engine/jit.ts:40-58)
    this.graph = (jit_cache: ExecItem[], input_rawbuffers: Buffer[], var_vals: Map<Variable, number>) =>
      CUDAGraph.capture(this, jit_cache, input_rawbuffers, var_vals, async () => {
        for (const ji of jit_cache) await ji.run(var_vals)
      })
  }
  // awaited before every lower / run (engine/realize.ts:133,157): idempotent
  override init = async () => {
    if (!lib) lib = await env.dlopen(vars.get('JSGRAD_CUDA_LIB', 'libjsgrad_cuda.so')!, SYMBOLS) as unknown as Lib
    if (this.handle) return
    const o = out64()
    check(lib.symbols.jg_device_open(this.ordinal, o))
    this.handle = Deno.UnsafePointer.create(o[0])
  }
  override synchronize = async () => check(await lib!.symbols.jg_device_sync(this.handle))
}
