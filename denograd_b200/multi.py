"""Tensor parallelism for the Llama path — the working counterpart of jsgrad/multi.ts, which in the reference is a stub
(every function throws NotImplemented, jsgrad/multi.ts:4-61).  What the reference does define is *which axis* each
weight is split on (jsgrad/models/llama3.ts:239-249); `shard_plan` follows it with one deliberate difference, taken
from the workload definition (all-reduce only after the attention-output and FFN-down projections): wq/wk/wv are split
by heads on their output axis instead of their input axis, so attention needs no exchange at all.

One rank is one process with one GPU (`TensorParallel`), or all ranks live in one process as in the reference engine
(`TensorParallel.init_all`).  The only exchanges per layer are two fp32 all-reduces (after `wo` and `w2`), plus one
max-reduction of the packed greedy keys per step when the output layer is sharded over the vocabulary.  All of them
run over NVLink peer memory once `open_peers` has mapped the ranks' exchange buffers:
  * 1-2 rows: the row-parallel projection only *pushes* its partial sums to the peers and the projection that consumes
    the sum (next norm + projection) adds them up in its prologue — nothing waits for another rank while idle;
  * up to 32 K values: one kernel in which every rank sends everything to everybody (flag-in-data entries);
  * up to 256 K values (a batch of 32-64 decode rows): a two-shot kernel, each rank reducing 1/world of the values
    straight out of the peers' partial-sum buffers;
  * beyond that (prompt chunks), or when a peer's memory cannot be mapped: NCCL all-reduce + a separate add.
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


def shard_plan(p: dict, rank: int, world: int, tied: bool, int8: bool = False) -> dict[str, Shard]:
    """Per-rank windows of every weight of architecture `p` (MODEL_PARAMS[...]['args'] layout).  With `int8` every
    weight also has a `.scale` entry: its per-output-row scales follow the rows of the weight's window (all rows,
    replicated, for the row-parallel wo / w2, whose windows span every output row).

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
    if int8:
        for name, sh in list(plan.items()):
            plan[name.replace(".weight", ".scale")] = Shard(sh.seed_name.replace(".weight", ".scale"), sh.rows, 1, 1, sh.row0, 0)
    return plan


def exchange_via_torch(mine: bytes) -> list[bytes]:
    """All-gather of one small byte string per rank through an initialised torch.distributed process group."""
    import torch.distributed as dist
    out: list = [None] * dist.get_world_size()
    dist.all_gather_object(out, mine)
    return out


def exchange_via_directory(path: str, rank: int, world: int, tag: str = "ipc", timeout: float = 120.0):
    """The same through files in a directory every rank can see (host-side wait with a deadline)."""
    import time

    def exchange(mine: bytes) -> list[bytes]:
        tmp = os.path.join(path, f"{tag}_{rank}.tmp")
        with open(tmp, "wb") as f:
            f.write(mine)
        os.replace(tmp, os.path.join(path, f"{tag}_{rank}.bin"))
        out, deadline = [], time.time() + timeout
        for r in range(world):
            fn = os.path.join(path, f"{tag}_{r}.bin")
            while not os.path.exists(fn):
                if time.time() > deadline:
                    raise TimeoutError(f"rank {r} never published its {tag} handle")
                time.sleep(0.02)
            out.append(open(fn, "rb").read())
        return out

    return exchange


class TensorParallel:
    """Rank handle: NCCL communicator bound to this process's device stream."""

    def __init__(self, dev: CUDA, rank: int, world: int, unique_id: bytes | None, handle=None):
        self.dev, self.rank, self.world = dev, rank, world
        self.peer_capacity = 0  # fp32 elements the one-shot peer-memory exchange takes; 0 until open_peers succeeded
        self.twoshot_capacity = 0  # fp32 elements of the two-shot exchange (its partial sums live in the exchange buffer)
        self._partial_ptr = 0
        if handle is not None:  # made by init_all: buffers and peers are in place already
            self.handle = handle
            self._query_capacity()
            return
        self.handle = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128)
        ffi.call("jg_comm_init", dev.handle, nccl_library_path().encode(), buf, rank, world, C.byref(self.handle))

    @staticmethod
    def init_all(devs: list[CUDA]) -> "list[TensorParallel]":
        """All ranks in this process (one thread drives every device, as the reference engine does): devs[r] is rank
        r.  The exchange buffers are addressed directly; NCCL collectives need `group()` around the per-rank calls."""
        ffi.load()
        n = len(devs)
        arr = (C.c_void_p * n)(*[d.handle for d in devs])
        out = (C.c_void_p * n)()
        ffi.call("jg_comm_init_all", n, arr, nccl_library_path().encode(), out)
        return [TensorParallel(devs[r], r, n, None, handle=C.c_void_p(out[r])) for r in range(n)]

    class group:
        """`with TensorParallel.group(): ...` brackets NCCL collectives one thread issues for several ranks."""

        def __enter__(self):
            ffi.call("jg_comm_group_begin")

        def __exit__(self, *a):
            ffi.call("jg_comm_group_end")
            return False

    def _query_capacity(self) -> None:
        cap = C.c_uint64(0)
        ffi.call("jg_comm_peer_capacity", self.handle, C.byref(cap))
        # one-shot exchange: every rank sends its whole message to every peer, which pays off only while latency
        # dominates: up to 32 K values (128 KB)
        self.peer_capacity = min(int(cap.value), 32 * 1024)
        if self.peer_capacity > 0:
            ptr, n = C.c_uint64(0), C.c_uint64(0)
            ffi.call("jg_comm_peer_partial", self.handle, C.byref(ptr), C.byref(n))
            self._partial_ptr, self.twoshot_capacity = int(ptr.value), int(n.value)

    @staticmethod
    def unique_id() -> bytes:
        """128-byte NCCL id made by one rank; hand it to the others out of band (a torch.distributed broadcast,
        a file, an environment variable)."""
        ffi.load()
        buf = C.create_string_buffer(128)
        ffi.call("jg_comm_unique_id", nccl_library_path().encode(), buf)
        return buf.raw

    # ---------------------------------------------------------------- peer-memory exchange (small messages)
    def open_peers(self, exchange) -> bool:
        """Map every rank's exchange buffer over NVLink peer memory.  `exchange(mine: bytes) -> list[bytes]` gathers
        one 64-byte handle per rank in rank order (e.g. `exchange_via_torch`, `exchange_via_directory`).  Returns
        False, leaving the NCCL path in charge, when a peer's memory cannot be mapped."""
        buf = C.create_string_buffer(64)
        ffi.call("jg_comm_peer_export", self.handle, buf)
        handles = exchange(buf.raw)
        assert len(handles) == self.world and all(len(h) == 64 for h in handles)
        try:
            ffi.call("jg_comm_peer_open", self.handle, C.create_string_buffer(b"".join(handles), 64 * self.world))
        except ffi.JgError as e:
            if e.status != 95:  # anything but "not supported" is a real error
                raise
            return False
        self._query_capacity()
        return self.peer_capacity > 0

    def partial_tensor(self, rows: int, dim: int) -> Tensor | None:
        """fp32 [rows, dim] over the region of the exchange buffer the peers can read, for the partial sums of a
        row-parallel projection that the two-shot exchange reduces in place; None when it does not fit."""
        if rows * dim > self.twoshot_capacity or os.environ.get("JG_TP_TWOSHOT", "1") == "0":
            return None
        from .device import Buffer
        return Tensor(Buffer.external(self.dev, self._partial_ptr, rows * dim, "float32"), shape=(rows, dim))

    def reduce_into_residual(self, h: Tensor, part32: Tensor) -> None:
        """h <- h + half(sum over ranks of part32): one of the peer-memory kernels when the message fits, else NCCL + add."""
        n = part32.numel()
        if 0 < n <= self.peer_capacity:
            ffi.call("jg_peer_allreduce_residual", self.handle, h.ptr, part32.ptr, n)
        elif part32.ptr == self._partial_ptr and n <= self.twoshot_capacity and n % 4 == 0:
            ffi.call("jg_peer_allreduce2_residual", self.handle, h.ptr, n)
        else:
            self.all_reduce_sum(part32)
            self.dev.call("jg_residual_add_f32", h.ptr, part32.ptr, n)

    def split_rows(self, int8: bool) -> int:
        """Most rows for which a row-parallel projection only pushes its partial sums and the next projection gathers
        them (`linear_push` + the gathering projections).  Off unless JG_TP_SPLIT=1: on two GPUs the projection fused
        with the whole exchange measured 441 tok/s against 432 for the split form (8B, batch 1), whose gathering
        prologue costs a cluster barrier more than the NVLink wait it hides."""
        if self.peer_capacity <= 0 or os.environ.get("JG_TP_SPLIT", "") != "1":
            return 0
        return 8 if int8 else 2

    def linear_push(self, x: Tensor, lin, rows: int) -> None:
        """First half of h <- h + half(sum over ranks of lin(x)): project and push the partial sums, wait for nobody."""
        ffi.call("jg_tp_linear_push", self.handle, x.ptr, lin.weight.ptr, lin.scale_ptr, rows, lin.out_features, lin.in_features)

    def fused_rows(self, int8: bool) -> int:
        """Most rows for which a row-parallel projection runs fused with its exchange (`linear_into_residual`):
        the matrix-vector kernels win up to 2 rows of fp16 weights and serve int8 up to 8; 0 without peer memory."""
        if self.peer_capacity <= 0 or os.environ.get("JG_TP_FUSED", "1") == "0":
            return 0
        return 8 if int8 else 2

    def linear_into_residual(self, h: Tensor, x: Tensor, lin, rows: int) -> None:
        """h <- h + half(sum over ranks of lin(x)) in one launch per rank (projection + all-reduce + residual add)."""
        ffi.call("jg_linear_allreduce_residual", self.handle, h.ptr, x.ptr, lin.weight.ptr, lin.scale_ptr, rows,
                 lin.out_features, lin.in_features)

    def all_reduce_sum(self, t: Tensor) -> None:
        assert t.dtype == "float32"
        ffi.call("jg_allreduce_sum_f32", self.handle, t.ptr, t.numel())

    def all_reduce_max(self, t: Tensor) -> None:
        assert t.dtype == "uint64"
        if 0 < t.numel() * 2 <= self.peer_capacity and t.ptr % 16 == 0:
            ffi.call("jg_peer_allreduce_max_u64", self.handle, t.ptr, t.numel())
        else:
            ffi.call("jg_allreduce_max_u64", self.handle, t.ptr, t.numel())

    def close(self) -> None:
        """Destroy the communicator.  Captured steps keep references to its collectives and NCCL waits for them, so
        drop every model (and its graphs) that used this rank handle first, or simply leave it to process exit."""
        if self.handle:
            ffi.call("jg_comm_destroy", self.handle)
            self.handle = None
