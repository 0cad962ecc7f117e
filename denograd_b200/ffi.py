"""ctypes binding of libjsgrad_cuda.so — the Python twin of the Deno.dlopen symbol table in ts/ops_cuda.ts.

Every call goes through the C ABI declared in include/jsgrad_cuda.h with the same argument order and types the
TypeScript device uses; a non-zero status becomes an exception carrying jg_last_error(), the reference's convention
for device failures (jsgrad/runtime/ops_clang.ts:34-35,42).  There is no fallback: if the shared library is
missing or cannot be loaded, importing a symbol raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("JG_LIB") or os.path.join(_HERE, "lib", "libjsgrad_cuda.so")

JG_OK, JG_EIO, JG_ENOMEM, JG_EINVAL, JG_ENOTSUP, JG_ETIMEDOUT = 0, 5, 12, 22, 95, 110


class JgError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[jsgrad_cuda status {status}] {message}")
        self.status = status


class Props(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("total_mem", C.c_uint64), ("l2_bytes", C.c_uint64), ("max_smem_per_block", C.c_int32)]


class KvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "n_kv_heads", "head_dim", "page_size", "n_pages", "max_batch",
                                          "max_pages_per_seq", "n_heads", "n_split")]


class StepDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "dim", "hidden_dim", "n_heads", "vocab_size", "freqs_rows")] + \
               [("norm_eps", C.c_float), ("vocab_offset", C.c_int32)] + \
               [(n, C.c_uint64) for n in ("layers", "tok_embeddings", "out_norm", "output", "freqs_cis", "comm")] + \
               [("embed_rows", C.c_int64)]


_vp, _i32, _i64, _u64, _f32, _f64, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_double, C.c_size_t
_P = C.POINTER

# name -> argument types; every function returns int status except jg_last_error.
SIGNATURES: dict[str, list] = {
    "jg_device_count": [_P(_i32)],
    "jg_device_open": [_i32, _P(_vp)],
    "jg_device_close": [_vp],
    "jg_device_sync": [_vp],
    "jg_device_props": [_vp, _P(Props)],
    "jg_launch_count": [_vp, _P(_u64)],
    "jg_alloc": [_vp, _sz, _P(_u64)],
    "jg_free": [_vp, _u64],
    "jg_copyin": [_vp, _u64, _vp, _sz],
    "jg_copyout": [_vp, _vp, _u64, _sz],
    "jg_transfer": [_vp, _u64, _vp, _u64, _sz],
    "jg_memset": [_vp, _u64, _i32, _sz],
    "jg_copy": [_vp, _u64, _u64, _sz],
    "jg_host_alloc": [_sz, _P(_vp)],
    "jg_host_free": [_vp],
    "jg_copyin_async": [_vp, _u64, _vp, _sz],
    "jg_copyout_async": [_vp, _vp, _u64, _sz],
    "jg_timer_start": [_vp],
    "jg_timer_stop": [_vp, _P(_f64)],
    "jg_cuda_compile": [C.c_char_p, C.c_char_p, _P(_vp), _P(_u64)],
    "jg_cuda_image_free": [_vp],
    "jg_program_load": [_vp, C.c_char_p, _vp, _u64, _P(_vp)],
    "jg_program_call": [_vp, _vp, _i32, _vp, _i32, _vp, _vp],
    "jg_program_destroy": [_vp],
    "jg_graph_begin": [_vp],
    "jg_graph_end": [_vp, _P(_vp)],
    "jg_graph_launch": [_vp, _vp],
    "jg_graph_destroy": [_vp],
    "jg_embed": [_vp, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_rmsnorm": [_vp, _u64, _u64, _u64, _i32, _i32, _f32],
    "jg_linear": [_vp, _u64, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_norm_linear": [_vp, _u64, _u64, _u64, _f32, _u64, _u64, _i32, _i32, _i32],
    "jg_norm_swiglu": [_vp, _u64, _u64, _u64, _f32, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_swiglu": [_vp, _u64, _u64, _u64, _i64],
    "jg_norm_logits_argmax": [_vp, _u64, _u64, _u64, _u64, _f32, _u64, _u64, _i32, _i32, _i32],
    "jg_argmax_finalize": [_vp, _u64, _u64, _i32],
    "jg_argmax": [_vp, _u64, _u64, _i32, _i32],
    "jg_sample": [_vp, _u64, _u64, _u64, _u64, _i32, _i32, _f32, _i32, _f32, _f32, _f32],
    "jg_freqs_cis": [_vp, _u64, _i32, _i32, _f64],
    "jg_kvcache_create": [_vp, _P(KvDesc), _P(_vp)],
    "jg_kvcache_destroy": [_vp],
    "jg_kvcache_set_block_table": [_vp, _vp],
    "jg_kvcache_bytes": [_vp, _P(_u64)],
    "jg_rope_kvwrite": [_vp, _vp, _i32, _u64, _u64, _i32, _u64, _i32, _i32],
    "jg_attn_decode": [_vp, _vp, _i32, _u64, _u64, _u64, _i32, _i32],
    "jg_attn_decode_fused": [_vp, _vp, _i32, _u64, _u64, _u64, _i32, _u64, _i32, _i32],
    "jg_rope_kvwrite_rows": [_vp, _vp, _i32, _u64, _u64, _i32, _u64, _u64, _i32, _i32],
    "jg_attn_rows": [_vp, _vp, _i32, _u64, _u64, _u64, _u64, _i32, _i32],
    "jg_attn_chunk": [_vp, _vp, _i32, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_attn_decode_noalloc": [_vp, _u64, _u64, _u64, _u64, _u64, _u64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32],
    "jg_step_create": [_vp, _vp, _P(StepDesc), _P(_vp)],
    "jg_step_destroy": [_vp],
    "jg_step_run": [_vp, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_pos_advance": [_vp, _u64, _i32],
    "jg_dequant_i8_f16": [_vp, _u64, _u64, _u64, _i64, _i64],
    "jg_dequant_nf4_f16": [_vp, _u64, _u64, _u64, _i64, _i32],
    "jg_fill_normal_f16": [_vp, _u64, _u64, _u64, _u64, _f32],
    "jg_fill_uniform_i8": [_vp, _u64, _u64, _u64, _u64],
    "jg_fill_scale_f16": [_vp, _u64, _u64, _u64, _u64, _f32],
    "jg_fill_const_f16": [_vp, _u64, _u64, _f32],
    "jg_fill_normal_f16_2d": [_vp, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _f32],
    "jg_fill_uniform_i8_2d": [_vp, _u64, _u64, _u64, _u64, _u64, _u64, _u64],
    "jg_comm_unique_id": [C.c_char_p, _vp],
    "jg_comm_init": [_vp, C.c_char_p, _vp, _i32, _i32, _P(_vp)],
    "jg_comm_destroy": [_vp],
    "jg_allreduce_sum_f32": [_vp, _u64, _u64],
    "jg_allreduce_max_u64": [_vp, _u64, _u64],
    "jg_comm_peer_export": [_vp, _vp],
    "jg_comm_peer_open": [_vp, _vp],
    "jg_comm_peer_capacity": [_vp, _vp],
    "jg_peer_allreduce_residual": [_vp, _u64, _u64, _u64],
    "jg_peer_allreduce_max_u64": [_vp, _u64, _u64],
    "jg_linear_allreduce_residual": [_vp, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_tp_linear_push": [_vp, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_tp_norm_linear": [_vp, _u64, _u64, _u64, _u64, _f32, _u64, _u64, _i32, _i32, _i32],
    "jg_tp_norm_swiglu": [_vp, _u64, _u64, _u64, _u64, _f32, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_tp_norm_logits_argmax": [_vp, _u64, _u64, _u64, _u64, _u64, _f32, _u64, _u64, _i32, _i32, _i32, _i32],
    "jg_comm_peer_partial": [_vp, _P(_u64), _P(_u64)],
    "jg_peer_allreduce2_residual": [_vp, _u64, _u64],
    "jg_comm_init_all": [_i32, _P(_vp), C.c_char_p, _P(_vp)],
    "jg_comm_group_begin": [],
    "jg_comm_group_end": [],
    "jg_linear_partial": [_vp, _u64, _u64, _u64, _u64, _i32, _i32, _i32],
    "jg_residual_add_f32": [_vp, _u64, _u64, _i64],
    "jg_norm_logits_argmax_shard": [_vp, _u64, _u64, _u64, _u64, _f32, _u64, _u64, _i32, _i32, _i32, _i32],
}

_lib: C.CDLL | None = None


def load() -> C.CDLL:
    """dlopen the library and declare every symbol of the header; raises if the library or a symbol is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m denograd_b200.build` "
                          "(there is no CPU fallback for the CUDA device)")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = args
        fn.restype = C.c_int
    lib.jg_last_error.argtypes = []
    lib.jg_last_error.restype = C.c_char_p
    _lib = lib
    return lib


def last_error() -> str:
    return (load().jg_last_error() or b"").decode("utf-8", "replace")


def check(status: int) -> None:
    if status != JG_OK:
        raise JgError(status, last_error())


def call(name: str, *args) -> None:
    """Invoke one C entry point and raise on a non-zero status."""
    check(getattr(load(), name)(*args))
