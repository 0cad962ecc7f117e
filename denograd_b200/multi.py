"""Tensor parallelism for the Llama path — the working counterpart of jsgrad/multi.ts, which in the reference is a stub
(every function throws NotImplemented, jsgrad/multi.ts:4-61).  What the reference does define is *which axis* each
weight is split on (jsgrad/models/llama3.ts:239-249); `shard_plan` follows it with one deliberate difference, taken
from the workload definition (all-reduce only after the attention-output and FFN-down projections): wq/wk/wv are split
by heads on their output axis instead of their input axis, so attention needs no exchange at all.

One rank is one process with one GPU.  The only exchanges per layer are two in-place fp32 all-reduces (after `wo` and
`w2`), plus one max-reduction of the packed greedy keys per step when the output layer is sharded over the vocabulary.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

from . import ffi
from .device import CUDA, Tensor


def nccl_library_path() -> str:
    """The libnccl.so.2 shipped with PyTorch's wheels if present, else the loader's default."""
    try:
        import nvidia.nccl as n  # namespace package of the nvidia-nccl wheel
        base = os.path.dirname(n.__file__) if getattr(n, "__file__", None) else list(n.__path__)[0]
        p = os.path.join(base, "lib", "libnccl.so.2")
        if os.path.exists(p):
            return p
    except Exception:
        pass
    return "libnccl.so.2"


@dataclass(frozen=True)
class Shard:
    """Window of a full [rows_full, cols_full] tensor held by one rank, and the name whose seed fills it."""
    seed_name: str
    rows: int
    cols: int
    cols_full: int
    row0: int
    col0: int


def shard_plan(p: dict, rank: int, world: int, tied: bool) -> dict[str, Shard]:
    """Per-rank windows of every weight of architecture `p` (MODEL_PARAMS[...]['args'] layout).

    column-parallel (rows of the weight): wq / wk / wv by heads, w1 / w3, output by vocabulary rows;
    row-parallel (columns of the weight, all-reduce after): wo, w2; replicated: norms and the embedding table.
    """
    d, H, G = p["dim"], p["n_heads"], p["n_kv_heads"]
    hd, f, V = d // H, p["hidden_dim"], p["vocab_size"]
    for name, v in (("n_heads", H), ("n_kv_heads", G), ("hidden_dim", f), ("vocab_size", V)):
        if v % world:
            raise ValueError(f"{name}={v} is not divisible by the tensor-parallel world size {world}")
    Hl, Gl, fl, Vl = H // world, G // world, f // world, V // world
    plan: dict[str, Shard] = {}
    for l in range(p["n_layers"]):
        a, ff = f"layers.{l}.attention", f"layers.{l}.feed_forward"
        plan[f"{a}.wq.weight"] = Shard(f"{a}.wq.weight", Hl * hd, d, d, rank * Hl * hd, 0)
        plan[f"{a}.wk.weight"] = Shard(f"{a}.wk.weight", Gl * hd, d, d, rank * Gl * hd, 0)
        plan[f"{a}.wv.weight"] = Shard(f"{a}.wv.weight", Gl * hd, d, d, rank * Gl * hd, 0)
        plan[f"{a}.wo.weight"] = Shard(f"{a}.wo.weight", d, Hl * hd, H * hd, 0, rank * Hl * hd)
        plan[f"{ff}.w1.weight"] = Shard(f"{ff}.w1.weight", fl, d, d, rank * fl, 0)
        plan[f"{ff}.w3.weight"] = Shard(f"{ff}.w3.weight", fl, d, d, rank * fl, 0)
        plan[f"{ff}.w2.weight"] = Shard(f"{ff}.w2.weight", d, fl, f, 0, rank * fl)
    plan["output.weight"] = Shard("tok_embeddings.weight" if tied else "output.weight", Vl, d, d, rank * Vl, 0)
    return plan


class TensorParallel:
    """Rank handle: NCCL communicator bound to this process's device stream."""

    def __init__(self, dev: CUDA, rank: int, world: int, unique_id: bytes):
        self.dev, self.rank, self.world = dev, rank, world
        self.handle = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128)
        ffi.call("jg_comm_init", dev.handle, nccl_library_path().encode(), buf, rank, world, C.byref(self.handle))

    @staticmethod
    def unique_id() -> bytes:
        """128-byte NCCL id made by one rank; hand it to the others out of band (a torch.distributed broadcast,
        a file, an environment variable)."""
        ffi.load()
        buf = C.create_string_buffer(128)
        ffi.call("jg_comm_unique_id", nccl_library_path().encode(), buf)
        return buf.raw

    def all_reduce_sum(self, t: Tensor) -> None:
        assert t.dtype == "float32"
        ffi.call("jg_allreduce_sum_f32", self.handle, t.ptr, t.numel())

    def all_reduce_max(self, t: Tensor) -> None:
        assert t.dtype == "uint64"
        ffi.call("jg_allreduce_max_u64", self.handle, t.ptr, t.numel())

    def close(self) -> None:
        """Destroy the communicator.  Captured steps keep references to its collectives and NCCL waits for them, so
        drop every model (and its graphs) that used this rank handle first, or simply leave it to process exit."""
        if self.handle:
            ffi.call("jg_comm_destroy", self.handle)
            self.handle = None
