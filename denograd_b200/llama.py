"""Llama transformer on the CUDA device — Python mirror of jsgrad/models/llama.ts.

Class and method names follow the reference (Attention, FeedForward, TransformerBlock, Transformer, TinyJit,
precompute_freqs_cis, apply_rotary_emb, sample); each method issues the library's kernels through the C ABI instead of
building a lazy graph.  Two ways through a block exist and compute the same values:

  * the per-op path (``fused=False``): one kernel per reference op — RMSNorm, Linear x3, RoPE + cache write,
    attention, Linear + add, RMSNorm, Linear x2, SiLU*mul, Linear + add;
  * the fused path (default): RMSNorm folded into the QKV / gate-up / logits projections, residual adds and SwiGLU
    folded into the projection epilogues, greedy selection folded into the logits kernel.

A decode step (tokens [B,1], start_pos > 0) is captured once into a CUDA graph and replayed, the role TinyJit has
in the reference (jsgrad/models/llama.ts:199,214-219, jsgrad/engine/jit.ts:236-353); `start_pos` and the tokens live
in device memory so that the captured step serves every position.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import ffi
from .device import CUDA, CUDAGraph, Device, Tensor
from .nn import Embedding, Linear, RMSNorm, _dev


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0, device=None) -> Tensor:
    """[end, dim/2, 2] table of (cos, sin), already cast to fp16 (jsgrad/models/llama.ts:10-14 and the cast at :205;
    the reference shapes it [1, end, 1, dim/2, 2])."""
    dev = _dev(device)
    t = Tensor.empty((end, dim // 2, 2), "float16", dev)
    dev.call("jg_freqs_cis", t.ptr, dim, end, float(theta))
    return t


class KVCache:
    """The model's paged K/V pool (what Attention.cache_kv is per layer in the reference, jsgrad/models/llama.ts:78-90)."""

    def __init__(self, dev: CUDA, n_layers: int, n_heads: int, n_kv_heads: int, head_dim: int, max_context: int,
                 max_batch: int, page_size: int = 64, n_split: int = 0):
        self.dev = dev
        self.page_size = page_size
        self.max_pages_per_seq = (max_context + page_size - 1) // page_size
        self.n_pages = self.max_pages_per_seq * max_batch
        self.max_batch = max_batch
        d = ffi.KvDesc(n_layers, n_kv_heads, head_dim, page_size, self.n_pages, max_batch, self.max_pages_per_seq,
                       n_heads, n_split)
        self.handle = C.c_void_p()
        ffi.call("jg_kvcache_create", dev.handle, C.byref(d), C.byref(self.handle))
        self.fused_attention = os.environ.get("JG_ATTN_FUSED", "1") != "0"  # one-launch decode attention

    def set_block_table(self, table: np.ndarray) -> None:
        table = np.ascontiguousarray(table, dtype=np.int32)
        assert table.shape == (self.max_batch, self.max_pages_per_seq), table.shape
        ffi.call("jg_kvcache_set_block_table", self.handle, table.ctypes.data_as(C.c_void_p))

    def nbytes(self) -> int:
        out = C.c_uint64(0)
        ffi.call("jg_kvcache_bytes", self.handle, C.byref(out))
        return out.value

    def close(self) -> None:
        if self.handle:
            ffi.call("jg_kvcache_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            if self.dev.handle is not None:
                self.close()
        except Exception:
            pass


def apply_rotary_emb_kvwrite(qkv: Tensor, freqs_cis: Tensor, pos: Tensor, kv: KVCache, layer: int, n_heads: int) -> None:
    """apply_rotary_emb on the Q and K slices of `qkv` plus the cache assignment (jsgrad/models/llama.ts:23-32,87)."""
    qkv.dev.call("jg_rope_kvwrite", kv.handle, layer, qkv.ptr, freqs_cis.ptr, freqs_cis.shape[0], pos.ptr,
                 qkv.numel() // qkv.shape[-1], n_heads)


class Attention:
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int | None, max_context: int, linear=Linear, device=None,
                 head_dim: int | None = None):
        # under tensor parallelism n_heads / n_kv_heads are this rank's share and head_dim is given explicitly
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads if n_kv_heads is not None else n_heads
        self.head_dim = head_dim if head_dim is not None else dim // n_heads
        self.n_rep = self.n_heads // self.n_kv_heads
        self.max_context = max_context
        dev = _dev(device)
        q_out, kv_out = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        # wq|wk|wv share one allocation so that the three projections run as one pass over contiguous rows (the
        # reference's WQKV option concatenates them the same way, jsgrad/models/llama.ts:63-66); each Linear's
        # weight is a row view of it.
        self._wqkv = linear(dim, q_out + 2 * kv_out, False, device=dev)
        self.wq = linear(dim, q_out, False, **self._wqkv.row_views(0, q_out))
        self.wk = linear(dim, kv_out, False, **self._wqkv.row_views(q_out, q_out + kv_out))
        self.wv = linear(dim, kv_out, False, **self._wqkv.row_views(q_out + kv_out, q_out + 2 * kv_out))
        self.wo = linear(q_out, dim, False, device=dev)
        self._kv: KVCache | None = None
        self._layer = 0

    def call(self, x: Tensor, pos: Tensor, freqs_cis: Tensor, mask=None, residual: Tensor | None = None,
             out: Tensor | None = None, qkv: Tensor | None = None, attn: Tensor | None = None) -> Tensor:
        """x: already-normalised rows [B, 1, dim]; pos: device int32 [B] (the `start_pos` variable)."""
        if mask is not None:
            raise NotImplementedError("multi-token calls are fed one position at a time on this device")
        B = x.numel() // x.shape[-1]
        xqkv = self._wqkv.call(x, out=qkv)  # xq | xk | xv
        apply_rotary_emb_kvwrite(xqkv, freqs_cis, pos, self._kv, self._layer, self.n_heads)
        a = attn if attn is not None else Tensor.empty((B, self.n_heads * self.head_dim), "float16", x.dev)
        x.dev.call("jg_attn_decode", self._kv.handle, self._layer, a.ptr, xqkv.ptr, pos.ptr, B, self.n_heads)
        return self.wo.call(a, residual=residual, out=out)

    __call__ = call


class FeedForward:
    def __init__(self, dim: int, hidden_dim: int, linear=Linear, device=None):
        self.w1 = linear(dim, hidden_dim, False, device=device)
        self.w2 = linear(hidden_dim, dim, False, device=device)
        self.w3 = linear(dim, hidden_dim, False, device=device)  # the gate in Gated Linear Unit

    def call(self, x: Tensor, residual: Tensor | None = None, out: Tensor | None = None) -> Tensor:
        g, u = self.w1.call(x), self.w3.call(x)
        x.dev.call("jg_swiglu", g.ptr, g.ptr, u.ptr, g.numel())  # w1(x).silu() * w3(x), in place on g
        return self.w2.call(g, residual=residual, out=out)

    __call__ = call


class TransformerBlock:
    def __init__(self, dim: int, hidden_dim: int, n_heads: int, n_kv_heads: int | None, norm_eps: float, max_context: int,
                 linear=Linear, feed_forward=FeedForward, device=None, head_dim: int | None = None):
        self.attention = Attention(dim, n_heads, n_kv_heads, max_context, linear, device=device, head_dim=head_dim)
        self.feed_forward = feed_forward(dim, hidden_dim, linear, device=device)
        self.attention_norm = RMSNorm(dim, norm_eps, device=device)
        self.ffn_norm = RMSNorm(dim, norm_eps, device=device)

    def call(self, x: Tensor, pos: Tensor, freqs_cis: Tensor, mask=None) -> Tensor:
        """Per-op path: h = x + attention(attention_norm(x)); return h + feed_forward(ffn_norm(h))."""
        h = self.attention.call(self.attention_norm.call(x), pos, freqs_cis, mask, residual=x)
        return self.feed_forward.call(self.ffn_norm.call(h), residual=h)

    def call_fused(self, ws: "_Workspace", pos: Tensor, freqs_cis: Tensor, tp=None) -> None:
        """Same block on the workspace `ws` (h is updated in place) with the norms and elementwise ops folded into
        the projection kernels."""
        a, f, dev, B = self.attention, self.feed_forward, ws.h.dev, ws.B
        d = ws.h.shape[-1]
        wqkv = a._wqkv
        int8 = wqkv.scale_ptr != 0
        # tensor parallelism, 1-2 rows: the row-parallel projections push their partial sums and the norm + projection
        # that follows gathers them (and writes the new residual stream into the workspace's other h buffer)
        split = tp is not None and B <= tp.split_rows(int8)
        # from 3 rows on (fp16 weights) normalise into ws.xn and project on the tensor cores; the fused-norm kernels
        # stream through the CUDA cores and only keep up with the weights for 1-2 rows (int8 weights: never)
        big = _norm_first(B, int8, d) and not split
        if split and ws.pending:  # the previous block's w2 left its sum on the wire
            h_in, h_out = ws.flip()
            ffi.call("jg_tp_norm_linear", tp.handle, ws.qkv.ptr, h_out.ptr, h_in.ptr, self.attention_norm.weight.ptr,
                     self.attention_norm.eps, wqkv.weight.ptr, wqkv.scale_ptr, B, wqkv.out_features, d)
        elif big:
            self.attention_norm.call(ws.h, out=ws.xn)
            dev.call("jg_linear", ws.qkv.ptr, ws.xn.ptr, wqkv.weight.ptr, wqkv.scale_ptr, 0, B, wqkv.out_features, d)
        else:
            dev.call("jg_norm_linear", ws.qkv.ptr, ws.h.ptr, self.attention_norm.weight.ptr, self.attention_norm.eps,
                     wqkv.weight.ptr, wqkv.scale_ptr, B, wqkv.out_features, d)
        if a._kv.fused_attention:
            try:  # RoPE + cache write + attention in one cluster launch
                dev.call("jg_attn_decode_fused", a._kv.handle, a._layer, ws.attn.ptr, ws.qkv.ptr, freqs_cis.ptr,
                         freqs_cis.shape[0], pos.ptr, B, a.n_heads)
            except ffi.JgError as e:
                if e.status != ffi.JG_ENOTSUP:
                    raise
                a._kv.fused_attention = False  # context slice too long for shared memory: use the split kernels
        if not a._kv.fused_attention:
            apply_rotary_emb_kvwrite(ws.qkv, freqs_cis, pos, a._kv, a._layer, a.n_heads)
            dev.call("jg_attn_decode", a._kv.handle, a._layer, ws.attn.ptr, ws.qkv.ptr, pos.ptr, B, a.n_heads)
        self._row_parallel(a.wo, ws.attn, ws, tp, split=split)
        if split:
            h_in, h_out = ws.flip()
            ffi.call("jg_tp_norm_swiglu", tp.handle, ws.ffn.ptr, h_out.ptr, h_in.ptr, self.ffn_norm.weight.ptr, self.ffn_norm.eps,
                     f.w1.weight.ptr, f.w1.scale_ptr, f.w3.weight.ptr, f.w3.scale_ptr, B, f.w1.out_features, d)
        elif big:
            self.ffn_norm.call(ws.h, out=ws.xn)
            dev.call("jg_norm_swiglu", ws.ffn.ptr, ws.xn.ptr, 0, self.ffn_norm.eps, f.w1.weight.ptr,
                     f.w1.scale_ptr, f.w3.weight.ptr, f.w3.scale_ptr, B, f.w1.out_features, d)
        else:
            dev.call("jg_norm_swiglu", ws.ffn.ptr, ws.h.ptr, self.ffn_norm.weight.ptr, self.ffn_norm.eps, f.w1.weight.ptr,
                     f.w1.scale_ptr, f.w3.weight.ptr, f.w3.scale_ptr, B, f.w1.out_features, d)
        self._row_parallel(f.w2, ws.ffn, ws, tp, split=split)

    @staticmethod
    def _row_parallel(lin, x: Tensor, ws: "_Workspace", tp, w=None, split: bool = False) -> None:
        """h <- h + lin(x).  On one device the add is the projection's epilogue; under tensor parallelism `lin` holds a
        K-slice, so its fp32 partial sums are all-reduced first and rounded + added afterwards.  `w` = (weight pointer,
        scale pointer) replaces lin's own (a dequantised copy of int8 weights).  With `split` only the first half of
        the exchange happens here: the sum is completed by the next projection's prologue (ws.pending says so)."""
        wp, sp = w if w is not None else (lin.weight.ptr, lin.scale_ptr)
        dev = ws.h.dev
        if split:
            tp.linear_push(x, lin, ws.B)
            ws.pending = True
            return
        if tp is None:
            dev.call("jg_linear", ws.h.ptr, x.ptr, wp, sp, ws.h.ptr, ws.B, lin.out_features, lin.in_features)
            return
        if w is None and ws.B <= tp.fused_rows(lin.scale_ptr != 0):
            tp.linear_into_residual(ws.h, x, lin, ws.B)
            return
        dev.call("jg_linear_partial", ws.part32.ptr, x.ptr, wp, sp, ws.B, lin.out_features, lin.in_features)
        tp.reduce_into_residual(ws.h, ws.part32)

    __call__ = call


_alpha_counter: dict[tuple, Tensor] = {}  # the reference keeps one module-level counter (jsgrad/models/llama.ts:130)


def sample(logits: Tensor, temp: float, k: int, p: float, af: float, ap: float, u: Tensor | None = None,
           out: Tensor | None = None) -> Tensor:
    """`sample` (jsgrad/models/llama.ts:131-185) per row of fp16 logits [rows, V]: argmax with the lowest index among
    equals when temp < 1e-6, else alpha penalties, softmax(logits / temp), top-k, approximate top-p and the multinomial
    draw in one kernel.  `u`: float32 [rows] uniform samples for the draw; by default they come from the restated
    Tensor.rand stream (denograd_b200.rand, seeded by rand.manual_seed)."""
    V = logits.shape[-1]
    rows = logits.numel() // V
    if p < 0 or p > 1:
        raise ValueError("p must be between 0 and 1")
    if k < 0 or k > V:
        raise ValueError("k must be between 0 and numel")
    out = out if out is not None else Tensor.empty((rows,), "int32", logits.dev)
    if temp < 1e-6:
        logits.dev.call("jg_argmax", out.ptr, logits.ptr, rows, V)
        return out
    if u is None:
        from . import rand
        u = Tensor(rand.rand(rows, logits.dev.device), device=logits.dev)
    counter_ptr = 0
    if af or ap:
        key = (logits.dev.device, rows, V)
        if key not in _alpha_counter:
            _alpha_counter[key] = Tensor.zeros((rows, V), "int32", logits.dev)
        counter_ptr = _alpha_counter[key].ptr
    logits.dev.call("jg_sample", out.ptr, logits.ptr, u.ptr, counter_ptr, rows, V, float(temp), int(k), float(p), float(af), float(ap))
    return out


def _norm_first(rows: int, int8: bool, dim: int = 0) -> bool:
    """Whether RMSNorm runs as its own kernel ahead of a projection.  The matrix-vector kernels fuse the norm into
    their prologue; the tensor-core kernels take normalised rows: fp16 weights from 3 rows on; int8 weights beyond 1
    row, or when `rows` rows of `dim` halves are too many to stay in shared memory next to a second CTA (the int8
    matrix-vector kernel keeps them there; `dim` = 0: unknown, normalise first)."""
    if int8:
        if os.environ.get("JG_W8_RESIDENT_X") is not None:  # the kernel is switched off: k-tiled tensor-core kernel
            return rows > 8 or os.environ.get("JG_W8_MMA", "1") != "0"
        max_m = int(os.environ.get("JG_W8_RESIDENT_MAX_M", "1"))
        return rows > max_m or dim <= 0 or dim % 512 != 0 or 2 * (rows * (2 * dim + 16) + 4096) > 228 * 1024
    return rows >= 3


class _Workspace:
    """Activation buffers of one decode step for a fixed batch size (what the memory planner would assign,
    jsgrad/engine/memory.ts:8-58): reused by every layer and every step, so a captured step never allocates."""

    def __init__(self, dev: CUDA, B: int, dim: int, qkv_dim: int, q_dim: int, hidden: int, vocab: int, tp=None):
        """`vocab` = 0 leaves out the logits (a multi-position chunk only projects its last rows, elsewhere)."""
        self.B = B
        self._dev = dev
        self.tokens = Tensor.zeros((B,), "int32", dev)
        self.pos = Tensor.zeros((B,), "int32", dev)
        self.hist = None  # picks of a run of steps made by one launch ([n_steps][B] int32)
        self.seq = Tensor.zeros((B,), "int32", dev)  # row -> sequence, for multi-position chunks
        # the residual stream; under tensor parallelism a second buffer, because the projection that completes a pushed
        # all-reduce writes the new stream while other CTAs still read the old one (`flip`)
        self._h = [Tensor.empty((B, dim), "float16", dev)]
        if tp is not None:
            self._h.append(Tensor.empty((B, dim), "float16", dev))
        self.cur = 0
        self.pending = False  # a row-parallel projection has pushed partial sums that nobody has gathered yet
        self.xn = Tensor.empty((B, dim), "float16", dev)
        self.qkv = Tensor.empty((B, qkv_dim), "float16", dev)
        self.attn = Tensor.empty((B, q_dim), "float16", dev)
        self.ffn = Tensor.empty((B, hidden), "float16", dev)
        self.logits = Tensor.empty((B, vocab), "float16", dev) if vocab else None
        self.key = Tensor.zeros((B,), "uint64", dev)
        self.next_tokens = Tensor.zeros((B,), "int32", dev)
        # fp32 partial sums of a row-parallel projection: inside the exchange buffer when they fit there, so that the
        # peers can read them (two-shot exchange)
        self.part32 = (tp.partial_tensor(B, dim) if tp is not None else None) or Tensor.empty((B, dim), "float32", dev)
        # page-locked staging for the per-step token / position upload and the result read-back
        self._pinned = C.c_void_p()
        ffi.call("jg_host_alloc", 3 * 4 * B, C.byref(self._pinned))
        arr = np.ctypeslib.as_array((C.c_int32 * (3 * B)).from_address(self._pinned.value))
        self.h_tokens, self.h_pos, self.h_next = arr[:B], arr[B:2 * B], arr[2 * B:]

    @property
    def h(self) -> Tensor:
        return self._h[self.cur]

    def flip(self) -> tuple[Tensor, Tensor]:
        """(stream before the pending sum, buffer that receives the stream after it); the latter becomes `h`."""
        old = self._h[self.cur]
        self.cur ^= 1
        self.pending = False
        return old, self._h[self.cur]

    def __del__(self):
        try:
            if self._pinned and self._dev.handle is not None:
                ffi.call("jg_host_free", self._pinned)
        except Exception:
            pass


class _StepPlan:
    """Handle of the single-kernel decode step of one model (jg_step_create): the table of the layers' tensors and
    the kernel's scratch.  The tensors' addresses are fixed at creation, like those a captured graph holds."""

    def __init__(self, model: "Transformer"):
        rows = []
        for layer in model.layers:
            a, f = layer.attention, layer.feed_forward
            rows.append([layer.attention_norm.weight.ptr, a._wqkv.weight.ptr, a.wo.weight.ptr, layer.ffn_norm.weight.ptr,
                         f.w1.weight.ptr, f.w3.weight.ptr, f.w2.weight.ptr])
        table = np.ascontiguousarray(rows, dtype=np.uint64)
        tp = model._tp  # tensor parallelism: the dimensions are this rank's shares, the exchanges happen inside the kernel
        comm = tp.handle.value if tp is not None else 0
        d = ffi.StepDesc(len(model.layers), model.dim, model.hidden_dim, model.n_heads, model.vocab_local,
                         model.freqs_cis.shape[0], model.norm.eps, model.vocab_offset, table.ctypes.data,
                         model.tok_embeddings.weight.ptr, model.norm.weight.ptr, model.output.weight.ptr, model.freqs_cis.ptr,
                         comm or 0, model.vocab_size)
        self._dev = model.dev
        self.handle = C.c_void_p()
        ffi.call("jg_step_create", model.dev.handle, model._kv.handle, C.byref(d), C.byref(self.handle))

    def __del__(self):
        try:
            if self.handle and self._dev.handle is not None:
                ffi.call("jg_step_destroy", self.handle)
                self.handle = None
        except Exception:
            pass


class TinyJit:
    """Call 0 runs eagerly, call 1 runs while being captured, later calls replay the capture
    (jsgrad/engine/jit.ts:273-353).  The wrapped function must read its varying inputs from device memory."""

    def __init__(self, fxn, dev: CUDA):
        self.fxn, self.dev = fxn, dev
        self.cnt = 0
        self.graph: CUDAGraph | None = None

    def reset(self) -> None:
        self.cnt, self.graph = 0, None

    def call(self, *args):
        if self.cnt == 0:
            self.fxn(*args)
        elif self.cnt == 1:
            g = CUDAGraph(self.dev)
            with g:
                self.fxn(*args)
            self.graph = g
            g.launch()  # a captured launch list has not run yet
        else:
            self.graph.launch()
        self.cnt += 1

    __call__ = call


class Transformer:
    def __init__(self, dim: int, hidden_dim: int, n_heads: int, n_layers: int, norm_eps: float, vocab_size: int,
                 linear=Linear, embedding=Embedding, n_kv_heads: int | None = None, rope_theta: float = 10000,
                 max_context: int = 1024, jit: bool = True, feed_forward=FeedForward, device=None, max_batch: int = 1,
                 page_size: int = 64, tied_output: bool = False, fused: bool = True, n_split: int = 0, tp=None):
        dev = _dev(device)
        self.dev, self.dim, self.vocab_size = dev, dim, vocab_size
        self.head_dim = dim // n_heads
        n_kv_heads = n_kv_heads if n_kv_heads is not None else n_heads
        self._tp = tp
        self._shards = None
        self.vocab_offset = 0
        if tp is not None and not fused:
            raise NotImplementedError("tensor parallelism runs on the fused block path")
        if tp is not None:
            # this rank's share (denograd_b200.multi.shard_plan): heads, kv heads, FFN width and vocabulary rows
            from .multi import shard_plan
            full = {"dim": dim, "n_heads": n_heads, "n_kv_heads": n_kv_heads, "hidden_dim": hidden_dim,
                    "vocab_size": vocab_size, "n_layers": n_layers}
            self._shards = shard_plan(full, tp.rank, tp.world, tied_output, int8=embedding is not Embedding)
            n_heads, n_kv_heads, hidden_dim = n_heads // tp.world, n_kv_heads // tp.world, hidden_dim // tp.world
            self.vocab_offset = tp.rank * (vocab_size // tp.world)
        self.hidden_dim = hidden_dim
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.vocab_local = vocab_size // tp.world if tp is not None else vocab_size
        self.max_context, self.max_batch, self.fused = max_context, max_batch, fused
        self.layers = [TransformerBlock(dim, hidden_dim, n_heads, n_kv_heads, norm_eps, max_context, linear, feed_forward,
                                        device=dev, head_dim=self.head_dim)
                       for _ in range(n_layers)]
        self.norm = RMSNorm(dim, norm_eps, device=dev)
        self.tok_embeddings = embedding(vocab_size, dim, device=dev)
        if tp is not None:
            # rows [vocab_offset, +vocab_local) of the full matrix (of the embedding table when tied); the embedding
            # table itself stays whole on every rank
            self.output = (Linear if embedding is Embedding else linear)(dim, self.vocab_local, False, device=dev)
        elif tied_output:
            # output.weight is the embedding table itself (Llama-3.2 1B/3B; for quantised embeddings the reference
            # ties them as well, jsgrad/models/llama3.ts:55-58)
            if embedding is Embedding:
                self.output = Linear(dim, vocab_size, False, weight=self.tok_embeddings.weight)
            else:
                self.output = linear(dim, vocab_size, False, weight=self.tok_embeddings.weight, scale=self.tok_embeddings.scale)
        else:
            self.output = Linear(dim, vocab_size, False, device=dev) if embedding is Embedding else linear(dim, vocab_size, False, device=dev)
        self.freqs_cis = precompute_freqs_cis(self.head_dim, self.max_context * 2, rope_theta, device=dev)
        self._kv_args = (n_layers, n_heads, self.n_kv_heads, self.head_dim, max_context, max_batch, page_size, n_split)
        self._kv = KVCache(dev, *self._kv_args)
        for i, layer in enumerate(self.layers):
            layer.attention._kv, layer.attention._layer = self._kv, i
        self._ws: dict[int, _Workspace] = {}
        self._jit_enabled = jit
        self._forward_jit: dict[int, TinyJit] = {}
        self._loop_graph: dict[int, CUDAGraph] = {}
        self._step_plan = None  # None: not tried yet, False: this model keeps the launch-per-op step

    def new_cache(self) -> None:
        """An empty (all-zero) KV cache in place of the current one, as a newly built model has (the lazily created
        Attention.cache_kv of jsgrad/models/llama.ts:78-90).  Everything that holds the old cache's addresses goes
        with it: the captured decode graphs and the single-kernel step plan are rebuilt on their next use."""
        self._forward_jit.clear()
        self._loop_graph.clear()
        self._step_plan = None
        self.dev.synchronize()
        old, self._kv = self._kv, KVCache(self.dev, *self._kv_args)
        for layer in self.layers:
            layer.attention._kv = self._kv
        old.close()

    # ------------------------------------------------------------------------------------------ internals
    def _workspace(self, B: int, rows: bool = False) -> _Workspace:
        """Workspace for B activation rows; `rows` marks a multi-position chunk (more rows than sequences allowed)."""
        if B > self.max_batch and not rows:
            raise ValueError(f"batch {B} exceeds max_batch {self.max_batch}")
        key = B if (not rows or B <= self.max_batch) else -B  # chunks beyond the batch limit carry no logits buffer
        if key not in self._ws:
            qkv_dim = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
            self._ws[key] = _Workspace(self.dev, B, self.dim, qkv_dim, self.n_heads * self.head_dim, self.hidden_dim,
                                       self.vocab_local if key > 0 else 0, tp=self._tp)
        return self._ws[key]

    def _single_kernel_step(self, B: int):
        """The step plan (jg_step_create) when this model and batch can run the decode step as one persistent kernel:
        fp16 weights, fused path, one device, 1-2 rows, a shape the kernel is instantiated for; else None."""
        if B > 2 or self._step_plan is False:
            return None
        if self._step_plan is None:
            self._step_plan = False
            a0 = self.layers[0].attention
            # tensor parallel: measured ahead of the launch-per-op step on 2 and 4 GPUs (506 against 443, 637 against 588
            # tok/s on the 8B shapes), behind it on 8 (646 against 679), where the two exchanges per layer outweigh the
            # rank's 8 us of weights; JG_STEP_KERNEL_TP=1 / 0 forces it on / off
            want_tp = os.environ.get("JG_STEP_KERNEL_TP", "1" if (self._tp is None or self._tp.world <= 4) else "0") != "0"
            tp_ok = self._tp is None or (self._tp.peer_capacity > 0 and want_tp)
            plain = (self.fused and tp_ok and os.environ.get("JG_STEP_KERNEL", "1") != "0"
                     and type(a0.wo) is Linear and type(self.output) is Linear and type(self.tok_embeddings) is Embedding
                     and type(self.layers[0].feed_forward) is FeedForward)
            if plain:
                try:
                    self._step_plan = _StepPlan(self)
                except ffi.JgError as e:
                    if e.status != ffi.JG_ENOTSUP:
                        raise
        return self._step_plan or None

    def _step(self, ws: _Workspace, advance: bool = False) -> None:
        """One token per row: reads ws.tokens / ws.pos, writes ws.logits and ws.next_tokens.  With `advance` the step
        also feeds its own output back (tokens <- next, pos += 1) so that it can be replayed with no host input."""
        dev, B = self.dev, ws.B
        cur0 = ws.cur
        plan = self._single_kernel_step(B)
        if plan is not None:  # the whole step as one persistent kernel
            ffi.call("jg_step_run", plan.handle, ws.tokens.ptr, ws.pos.ptr, ws.h.ptr, ws.qkv.ptr, ws.attn.ptr, ws.ffn.ptr,
                     ws.logits.ptr, ws.next_tokens.ptr, B, 1, 1 if advance else 0)
            return
        self.tok_embeddings.call(ws.tokens, out=ws.h)
        if self.fused:
            for layer in self.layers:
                layer.call_fused(ws, ws.pos, self.freqs_cis, self._tp)
            out = self.output
            if ws.pending:  # the last block's w2 pushed its sum: the output layer's prologue completes it
                h_in, h_out = ws.flip()
                ffi.call("jg_tp_norm_logits_argmax", self._tp.handle, ws.logits.ptr, ws.key.ptr, h_out.ptr, h_in.ptr,
                         self.norm.weight.ptr, self.norm.eps, out.weight.ptr, out.scale_ptr, B, self.vocab_local, self.dim,
                         self.vocab_offset)
                assert ws.cur == cur0, "a captured step must end on the residual buffer it started on"
            elif _norm_first(B, out.scale_ptr != 0, self.dim):
                self.norm.call(ws.h, out=ws.xn)
                dev.call("jg_norm_logits_argmax_shard", ws.logits.ptr, ws.key.ptr, ws.xn.ptr, 0, self.norm.eps,
                         out.weight.ptr, out.scale_ptr, B, self.vocab_local, self.dim, self.vocab_offset)
            else:
                dev.call("jg_norm_logits_argmax_shard", ws.logits.ptr, ws.key.ptr, ws.h.ptr, self.norm.weight.ptr, self.norm.eps,
                         out.weight.ptr, out.scale_ptr, B, self.vocab_local, self.dim, self.vocab_offset)
            if self._tp is not None:
                self._tp.all_reduce_max(ws.key)  # best (value, lowest global index) over the vocabulary shards
            dev.call("jg_argmax_finalize", ws.next_tokens.ptr, ws.key.ptr, B)
        else:
            h = ws.h
            for layer in self.layers:
                h = layer.call(h, ws.pos, self.freqs_cis, None)
            self.output.call(self.norm.call(h), out=ws.logits)
            dev.call("jg_argmax", ws.next_tokens.ptr, ws.logits.ptr, B, self.vocab_size)
        if advance:
            dev.call("jg_copy", ws.tokens.ptr, ws.next_tokens.ptr, 4 * B)
            dev.call("jg_pos_advance", ws.pos.ptr, B)

    # ------------------------------------------------------------------------------------------ reference API
    def forward(self, tokens, start_pos: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 0.8,
                alpha_f: float = 0.0, alpha_p: float = 0.0) -> Tensor:
        """Transformer.forward (jsgrad/models/llama.ts:201-213), eager.  tokens: int32 [B, S] (host array or Tensor).
        S > 1 runs in chunks of up to 2048 rows (batch x positions; 64 where a projection's shape keeps it off the
        tcgen05 kernel or the weights are int8): one pass over the weights per chunk, every row
        attending to the cache up to its own position — what the reference's additive causal mask (:208) computes.
        Returns the greedy next token of every batch row after the last position ([B] int32)."""
        toks = tokens.numpy() if isinstance(tokens, Tensor) else np.asarray(tokens, dtype=np.int32)
        B, S = toks.shape
        if start_pos + S > self.max_context:
            raise ValueError(f"start_pos {start_pos} + {S} tokens exceeds max_context {self.max_context}")
        ws = self._workspace(B)
        max_rows = self._max_chunk_rows()
        if S > 1 and self.fused and B <= max_rows and os.environ.get("JG_PREFILL", "rows") != "token":
            sc = max(1, max_rows // B)
            for s0 in range(0, S, sc):
                self._forward_rows(toks[:, s0:s0 + sc], start_pos + s0, last=(s0 + sc >= S))
            return self._pick(ws, temperature, top_k, top_p, alpha_f, alpha_p)
        for s in range(S):
            ws.tokens.assign(toks[:, s])
            ws.pos.assign(np.full((B,), start_pos + s, np.int32))
            self._step(ws)
        return self._pick(ws, temperature, top_k, top_p, alpha_f, alpha_p)

    def _pick(self, ws: _Workspace, temperature: float, top_k: int, top_p: float, alpha_f: float, alpha_p: float) -> Tensor:
        """The token of the last step: the greedy pick the logits kernel already made, or — temperature >= 1e-6 —
        `sample` over the step's logits (jsgrad/models/llama.ts:212)."""
        if temperature < 1e-6:
            return ws.next_tokens
        if self._tp is not None:
            raise NotImplementedError("stochastic sampling over a vocabulary-sharded output layer: gather the logits first")
        return sample(ws.logits, temperature, top_k, top_p, alpha_f, alpha_p, out=ws.next_tokens)

    def _max_chunk_rows(self) -> int:
        """Rows one projection call takes: 64 on the mma.sync kernel (int8 weights, or fp16 shapes off the tile grid),
        2048 when every projection of a block also fits the tcgen05 kernel (out features % 128, in features % 64)."""
        a, f = self.layers[0].attention, self.layers[0].feed_forward
        shapes = [(a._wqkv.out_features, self.dim), (self.dim, a.n_heads * self.head_dim),
                  (f.w1.out_features, self.dim), (self.dim, f.w1.out_features)]
        if all(n % 128 == 0 and k % 64 == 0 for n, k in shapes) and (self.output.scale_ptr == 0 or self._dequant_prefill()):
            return int(os.environ.get("JG_PREFILL_ROWS", "2048"))
        return 64

    @staticmethod
    def _dequant_prefill() -> bool:
        """int8 weights, more than 64 rows per chunk: the tcgen05 projection takes the int8 matrices and converts their
        tiles in shared memory (JG_W8_TC=0: each matrix is dequantised once per chunk into an fp16 scratch first — what
        the reference graph does for multi-row calls, jsgrad/models/llama3.ts:35); JG_W8_DEQUANT_PREFILL=0 keeps 64-row
        chunks on the mma.sync kernel instead."""
        return os.environ.get("JG_W8_DEQUANT_PREFILL", "1") != "0"

    def _fp16_weights(self, *lins):
        """(pointer, 0) per projection: the weights themselves when fp16, else their dequantised copy in the scratch."""
        if lins[0].scale_ptr == 0:
            return [(l.weight.ptr, 0) for l in lins]
        need = sum(l.out_features * l.in_features for l in lins)
        if getattr(self, "_dq_scratch", None) is None or self._dq_scratch.numel() < need:
            self._dq_scratch = Tensor.empty((need,), "float16", self.dev)
        out, off = [], 0
        for l in lins:
            ptr = self._dq_scratch.ptr + 2 * off
            self.dev.call("jg_dequant_i8_f16", ptr, l.weight.ptr, l.scale_ptr, l.out_features, l.in_features)
            out.append((ptr, 0))
            off += l.out_features * l.in_features
        return out

    def _forward_rows(self, toks: np.ndarray, start_pos: int, last: bool) -> None:
        """One chunk of a multi-position call: rows r = s * B + b (position-major), R = B * Sc.  With `last` the
        rows of the final position also go through the final norm, the output projection and greedy selection (the
        reference computes logits for every position and keeps the last, jsgrad/models/llama.ts:210)."""
        B, Sc = toks.shape
        R, dev, tp = B * Sc, self.dev, self._tp
        ws = self._workspace(R, rows=True)
        ws.tokens.assign(np.ascontiguousarray(toks.T).reshape(R))
        ws.pos.assign(np.repeat(np.arange(start_pos, start_pos + Sc, dtype=np.int32), B))
        ws.seq.assign(np.tile(np.arange(B, dtype=np.int32), Sc))
        self.tok_embeddings.call(ws.tokens, out=ws.h)
        d = self.dim
        # int8 weights and more rows than the mma.sync kernel takes: up to JG_W8_TC_ROWS rows the tcgen05 projection converts
        # the int8 tiles itself (every 256-row tile of activations converts the weight tiles again); beyond, and with
        # JG_W8_TC=0, it is given dequantised fp16 copies, made once per chunk
        tc_rows = 0 if os.environ.get("JG_W8_TC", "1") == "0" else int(os.environ.get("JG_W8_TC_ROWS", "768"))
        dq = R > 64 and self.output.scale_ptr != 0 and R > tc_rows

        def weights(*lins):
            return self._fp16_weights(*lins) if dq else [(l.weight.ptr, l.scale_ptr) for l in lins]

        for layer in self.layers:
            a, f = layer.attention, layer.feed_forward
            layer.attention_norm.call(ws.h, out=ws.xn)
            (wp, sp), = weights(a._wqkv)
            dev.call("jg_linear", ws.qkv.ptr, ws.xn.ptr, wp, sp, 0, R, a._wqkv.out_features, d)
            dev.call("jg_rope_kvwrite_rows", a._kv.handle, a._layer, ws.qkv.ptr, self.freqs_cis.ptr, self.freqs_cis.shape[0],
                     ws.pos.ptr, ws.seq.ptr, R, a.n_heads)
            if Sc >= 8 and os.environ.get("JG_ATTN_CHUNK", "1") != "0":  # tensor-core attention over the regular chunk
                dev.call("jg_attn_chunk", a._kv.handle, a._layer, ws.attn.ptr, ws.qkv.ptr, ws.pos.ptr, ws.seq.ptr, B, Sc, a.n_heads)
            else:
                dev.call("jg_attn_rows", a._kv.handle, a._layer, ws.attn.ptr, ws.qkv.ptr, ws.pos.ptr, ws.seq.ptr, R, a.n_heads)
            layer._row_parallel(a.wo, ws.attn, ws, tp, weights(a.wo)[0] if dq else None)
            layer.ffn_norm.call(ws.h, out=ws.xn)
            (w1p, s1p), (w3p, s3p) = weights(f.w1, f.w3)
            dev.call("jg_norm_swiglu", ws.ffn.ptr, ws.xn.ptr, 0, layer.ffn_norm.eps, w1p, s1p, w3p, s3p, R, f.w1.out_features, d)
            layer._row_parallel(f.w2, ws.ffn, ws, tp, weights(f.w2)[0] if dq else None)
        if last:
            wsb = self._workspace(B)  # logits / keys / next tokens live in the batch-sized workspace, as after a step
            h_last = ws.h.view_rows(R - B, R)
            xn_last = ws.xn.view_rows(R - B, R)
            self.norm.call(h_last, out=xn_last)
            out = self.output
            dev.call("jg_norm_logits_argmax_shard", wsb.logits.ptr, wsb.key.ptr, xn_last.ptr, 0, self.norm.eps,
                     out.weight.ptr, out.scale_ptr, B, self.vocab_local, self.dim, self.vocab_offset)
            if tp is not None:
                tp.all_reduce_max(wsb.key)
            dev.call("jg_argmax_finalize", wsb.next_tokens.ptr, wsb.key.ptr, B)

    def call(self, tokens, start_pos: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 0.8,
             alpha_f: float = 0.0, alpha_p: float = 0.0) -> Tensor:
        """Transformer.call (jsgrad/models/llama.ts:214-220): single-token calls after position 0 go through the jit."""
        toks = tokens.numpy() if isinstance(tokens, Tensor) else np.asarray(tokens, dtype=np.int32)
        B, S = toks.shape
        if S == 1 and self._jit_enabled and start_pos != 0:
            if start_pos + 1 > self.max_context:
                raise ValueError(f"start_pos {start_pos} + 1 exceeds max_context {self.max_context}")
            ws = self._workspace(B)
            ws.tokens.assign(toks[:, 0])
            ws.pos.assign(np.full((B,), start_pos, np.int32))
            if B not in self._forward_jit:
                self._forward_jit[B] = TinyJit(lambda: self._step(ws), self.dev)
            self._forward_jit[B].call()
            return self._pick(ws, temperature, top_k, top_p, alpha_f, alpha_p)
        return self.forward(toks, start_pos, temperature, top_k, top_p, alpha_f, alpha_p)

    __call__ = call

    def call_host(self, tokens: np.ndarray, start_pos: int) -> np.ndarray:
        """`call(...)` followed by reading the ids back (`.item()` in the reference's loop), for one new token per
        row after position 0, with the copies staged through page-locked memory: per step B*8 bytes go up (tokens and
        positions), the captured step runs, B*4 bytes come back.  tokens: int32 [B, 1] -> int32 [B]."""
        B = tokens.shape[0]
        if start_pos == 0 or not self._jit_enabled:
            return self.call(tokens, start_pos).numpy()
        if start_pos + 1 > self.max_context:
            raise ValueError(f"start_pos {start_pos} + 1 exceeds max_context {self.max_context}")
        ws = self._workspace(B)
        ws.h_tokens[:] = tokens.reshape(B)
        ws.h_pos[:] = start_pos
        dev = self.dev
        dev.call("jg_copyin_async", ws.tokens.ptr, ws.h_tokens.ctypes.data, 4 * B)
        dev.call("jg_copyin_async", ws.pos.ptr, ws.h_pos.ctypes.data, 4 * B)
        if B not in self._forward_jit:
            self._forward_jit[B] = TinyJit(lambda: self._step(ws), self.dev)
        self._forward_jit[B].call()
        dev.call("jg_copyout_async", ws.h_next.ctypes.data, ws.next_tokens.ptr, 4 * B)
        dev.synchronize()
        return ws.h_next.copy()

    # ------------------------------------------------------------------------------------------ device-resident loop
    def decode_loop(self, first_tokens, start_pos: int, n_steps: int, collect: bool = True,
                    resume: bool = False) -> np.ndarray | None:
        """Greedy-decode `n_steps` tokens per row with no host round trip between steps: the captured step feeds its
        own output back on the device.  Returns the generated ids [B, n_steps] (read back after the last step), or
        None when `collect` is false.  With `resume` the tokens and positions already on the device (left by the
        previous loop) are continued and `first_tokens` only gives the batch size; nothing is copied or synchronised,
        so a caller can time a run of steps with events."""
        toks = np.asarray(first_tokens, dtype=np.int32).reshape(-1)
        B = toks.shape[0]
        if start_pos + n_steps > self.max_context:
            raise ValueError(f"start_pos {start_pos} + {n_steps} steps exceeds max_context {self.max_context}")
        ws = self._workspace(B)
        if not resume:
            ws.tokens.assign(toks)
            ws.pos.assign(np.full((B,), start_pos, np.int32))
        plan = self._single_kernel_step(B)
        if plan is not None:
            # the persistent kernel loops over the steps itself: one launch for the whole run, picks land in `hist`
            if ws.hist is None or ws.hist.shape[0] < n_steps:
                ws.hist = Tensor.empty((max(n_steps, 64), B), "int32", self.dev)
            ffi.call("jg_step_run", plan.handle, ws.tokens.ptr, ws.pos.ptr, ws.h.ptr, ws.qkv.ptr, ws.attn.ptr, ws.ffn.ptr,
                     ws.logits.ptr, ws.hist.ptr, B, n_steps, 1)
            if not collect:
                return None
            out = ws.hist.numpy()[:n_steps].T.copy()
            self.dev.call("jg_copy", ws.next_tokens.ptr, ws.hist.ptr + 4 * B * (n_steps - 1), 4 * B)
            return out
        if B not in self._loop_graph:
            if resume:
                raise ValueError("nothing to resume: run decode_loop once without `resume` first")
            self._step(ws, advance=True)  # eager once (sizes smem attributes), then restore the inputs and capture
            ws.tokens.assign(toks)
            ws.pos.assign(np.full((B,), start_pos, np.int32))
            g = CUDAGraph(self.dev)
            with g:
                self._step(ws, advance=True)
            self._loop_graph[B] = g
        g = self._loop_graph[B]
        hist = Tensor.empty((n_steps, B), "int32", self.dev) if collect else None
        for i in range(n_steps):
            g.launch()
            if collect:
                self.dev.call("jg_copy", hist.ptr + 4 * B * i, ws.next_tokens.ptr, 4 * B)
        return hist.numpy().T.copy() if collect else None

    def last_logits(self, B: int) -> np.ndarray:
        """fp16 logits of the last step widened to fp32 (`.float()` at jsgrad/models/llama.ts:210), [B, vocab]."""
        return self._workspace(B).logits.numpy().astype(np.float32)
