"""The `CUDA` device: Python mirror of jsgrad's device plumbing for the hand-written sm_100a kernels.

Same roles and names as the reference so that the model code above it reads like jsgrad's:
  * ``CUDAAllocator``  — Allocator/LRUAllocator (jsgrad/runtime/allocator.ts:28-77): _alloc/_free/_copyin/_copyout/
                          _offset/_transfer over uint64 device addresses;
  * ``CUDA``           — Compiled (jsgrad/runtime/allocator.ts:166-191) registered under the name ``CUDA`` and looked
                          up through ``Device[...]`` like jsgrad/device.ts:10-43;
  * ``Buffer``         — jsgrad/device.ts:66-172 (allocate / view / copyin / copyout);
  * ``Tensor``         — only the slice of jsgrad/tensor.ts the Llama path touches: a realized fp16/int8/int32 buffer
                          with a shape.  There is no lazy graph here: every op is one of the library's kernels.
  * ``CUDAGraph``      — the GraphRunner a TinyJit batch becomes (jsgrad/engine/jit.ts:71-141);
  * ``CUDACompiler`` / ``CUDAProgram`` — Compiler / Program (jsgrad/runtime/allocator.ts:98-139, instance
                          jsgrad/runtime/ops_clang.ts:7-54) for CUDA C source such as the reference's CUDARenderer
                          emits (jsgrad/renderer/cstyle.ts:348-419): NVRTC to a cubin, loaded and launched on the
                          device's stream.  The way out for an AST without a hand-written kernel.
All device work goes through the C ABI in ``ffi`` (no torch, no CPU fallback).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Sequence

import numpy as np

from . import ffi

_DTYPE_SIZE = {"float16": 2, "int8": 1, "uint8": 1, "int32": 4, "float32": 4, "uint64": 8}
_NP = {"float16": np.float16, "int8": np.int8, "uint8": np.uint8, "int32": np.int32, "float32": np.float32, "uint64": np.uint64}


class CUDAAllocator:
    """LRU allocator over jg_alloc/jg_free (jsgrad/runtime/allocator.ts:53-77).  ``Buf`` is the device address."""

    def __init__(self, dev: "CUDA"):
        self.dev = dev  # BufferXfer reads `allocator.dev` on both sides (jsgrad/engine/realize.ts:126)
        self.cache: dict[int, list[int]] = {}
        self.allocated = 0

    def alloc(self, size: int) -> int:
        if size <= 0:
            raise ValueError(f"alloc size must be positve, getting {size}")
        c = self.cache.get(size)
        if c:
            return c.pop()
        return self._alloc(size)

    def free(self, opaque: int, size: int) -> None:
        self.cache.setdefault(size, []).append(opaque)

    def free_cache(self) -> None:
        for bufs in self.cache.values():
            for b in bufs:
                self._free(b)
        self.cache.clear()

    def _alloc(self, size: int) -> int:
        out = C.c_uint64(0)
        try:
            ffi.call("jg_alloc", self.dev.handle, size, C.byref(out))
        except ffi.JgError as e:
            if e.status != ffi.JG_ENOMEM or not self.cache:
                raise
            self.free_cache()  # LRUAllocator retries once after dropping its cache
            ffi.call("jg_alloc", self.dev.handle, size, C.byref(out))
        self.allocated += size
        return out.value

    def _free(self, opaque: int) -> None:
        ffi.call("jg_free", self.dev.handle, opaque)

    def _copyin(self, dest: int, src: np.ndarray) -> None:
        src = np.ascontiguousarray(src)
        ffi.call("jg_copyin", self.dev.handle, dest, src.ctypes.data_as(C.c_void_p), src.nbytes)

    def _copyout(self, dest: np.ndarray, src: int) -> None:
        assert dest.flags["C_CONTIGUOUS"]
        ffi.call("jg_copyout", self.dev.handle, dest.ctypes.data_as(C.c_void_p), src, dest.nbytes)

    @staticmethod
    def _offset(buf: int, size: int, offset: int) -> int:
        return buf + offset

    def _transfer(self, dest: int, src: int, sz: int, src_dev: "CUDA", dest_dev: "CUDA") -> None:
        ffi.call("jg_transfer", dest_dev.handle, dest, src_dev.handle, src, sz)


class CUDA:
    """Compiled device ``CUDA`` / ``CUDA:<n>``.  ``init`` is idempotent, as the engine awaits it before every use
    (jsgrad/engine/realize.ts:133,157)."""

    def __init__(self, device: str = "CUDA"):
        self.device = device
        self.ordinal = int(device.split(":")[1]) if ":" in device else 0
        self.handle: C.c_void_p | None = None
        self.allocator = CUDAAllocator(self)
        self.props: ffi.Props | None = None

    def init(self) -> "CUDA":
        if self.handle is None:
            ffi.load()
            h = C.c_void_p()
            ffi.call("jg_device_open", self.ordinal, C.byref(h))
            self.handle = h
            p = ffi.Props()
            ffi.call("jg_device_props", self.handle, C.byref(p))
            self.props = p
        return self

    def synchronize(self) -> None:
        ffi.call("jg_device_sync", self.handle)

    def launch_count(self) -> int:
        out = C.c_uint64(0)
        ffi.call("jg_launch_count", self.handle, C.byref(out))
        return out.value

    def timer_start(self) -> None:
        ffi.call("jg_timer_start", self.handle)

    def timer_stop(self) -> float:
        s = C.c_double(0.0)
        ffi.call("jg_timer_stop", self.handle, C.byref(s))
        return s.value

    def call(self, name: str, *args) -> None:
        """Program.call: run one kernel entry point on this device's stream."""
        ffi.call(name, self.handle, *args)

    def close(self) -> None:
        if self.handle is not None:
            self.allocator.free_cache()
            ffi.call("jg_device_close", self.handle)
            self.handle = None


class _DeviceRegistry:
    """``Device['CUDA:1']`` (jsgrad/device.ts:10-43): canonicalise the name, open each device once."""

    def __init__(self):
        self._opened: dict[str, CUDA] = {}
        self.DEFAULT = "CUDA"

    @staticmethod
    def canonicalize(device: str | None) -> str:
        d = (device or "CUDA").upper()
        name, _, ix = d.partition(":")
        if name != "CUDA":
            raise ValueError(f"unknown device {device!r}: this package registers the CUDA device only")
        return "CUDA" if ix in ("", "0") else f"CUDA:{int(ix)}"

    def __getitem__(self, device: str | None) -> CUDA:
        ix = self.canonicalize(device)
        if ix not in self._opened:
            self._opened[ix] = CUDA(ix).init()
        return self._opened[ix]

    get = __getitem__


Device = _DeviceRegistry()


class Buffer:
    """jsgrad/device.ts:66-172: a sized, typed region of device memory; ``view`` is an `_offset` sub-buffer."""

    def __init__(self, device: str | CUDA, size: int, dtype: str, base: "Buffer | None" = None, offset: int = 0):
        self.dev = device if isinstance(device, CUDA) else Device[device]
        self.size, self.dtype = size, dtype
        self.nbytes = size * _DTYPE_SIZE[dtype]
        self.base, self.offset = base, offset
        self._buf: int | None = None
        self._owned = True
        if base is not None:
            assert offset + self.nbytes <= base.nbytes, "view outside its base buffer"
            self._buf = CUDAAllocator._offset(base.ptr, self.nbytes, offset)

    @staticmethod
    def external(device: "str | CUDA", ptr: int, size: int, dtype: str) -> "Buffer":
        """A buffer over device memory somebody else owns (a region of the library's exchange buffer): never freed
        or cached by this allocator."""
        b = Buffer(device, size, dtype)
        b._buf, b._owned = ptr, False
        return b

    def allocate(self) -> "Buffer":
        if self._buf is None:
            self._buf = self.dev.allocator.alloc(self.nbytes)
        return self

    @property
    def ptr(self) -> int:
        if self._buf is None:
            self.allocate()
        return self._buf

    def view(self, size: int, dtype: str, offset: int) -> "Buffer":
        return Buffer(self.dev, size, dtype, base=self.base or self, offset=(self.offset if self.base else 0) + offset)

    def copyin(self, arr: np.ndarray) -> "Buffer":
        arr = np.ascontiguousarray(arr)
        if arr.nbytes != self.nbytes:
            raise ValueError(f"size mismatch, src.nbytes={arr.nbytes} != self.nbytes={self.nbytes}")
        self.dev.allocator._copyin(self.ptr, arr)
        return self

    def copyout(self, arr: np.ndarray) -> np.ndarray:
        if arr.nbytes != self.nbytes:
            raise ValueError(f"size mismatch, dst.nbytes={arr.nbytes} != self.nbytes={self.nbytes}")
        self.dev.allocator._copyout(arr, self.ptr)
        return arr

    def __del__(self):
        try:
            if self.base is None and self._owned and self._buf is not None and self.dev.handle is not None:
                self.dev.allocator.free(self._buf, self.nbytes)
        except Exception:
            pass


class Tensor:
    """A realized tensor on the CUDA device (the subset of jsgrad/tensor.ts the Llama path needs)."""

    def __init__(self, data, dtype: str | None = None, device: str | CUDA | None = None, shape: Sequence[int] | None = None):
        if isinstance(data, Buffer):
            self.buf, self.shape, self.dtype = data, tuple(shape), data.dtype
            return
        arr = np.asarray(data)
        if dtype is not None:
            arr = arr.astype(_NP[dtype])
        dtype = {np.dtype(np.float16): "float16", np.dtype(np.int8): "int8", np.dtype(np.uint8): "uint8", np.dtype(np.int32): "int32",
                 np.dtype(np.float32): "float32", np.dtype(np.uint64): "uint64"}.get(arr.dtype)
        if dtype is None:
            raise TypeError(f"dtype {arr.dtype} is not used on the CUDA device's Llama path")
        self.shape, self.dtype = tuple(arr.shape), dtype
        self.buf = Buffer(device or Device.DEFAULT, int(arr.size), dtype).allocate()
        self.buf.copyin(arr)

    @staticmethod
    def empty(shape: Sequence[int], dtype: str = "float16", device: str | CUDA | None = None) -> "Tensor":
        n = int(math.prod(shape))
        return Tensor(Buffer(device or Device.DEFAULT, n, dtype).allocate(), shape=shape)

    @staticmethod
    def zeros(shape: Sequence[int], dtype: str = "float16", device: str | CUDA | None = None) -> "Tensor":
        t = Tensor.empty(shape, dtype, device)
        ffi.call("jg_memset", t.dev.handle, t.ptr, 0, t.nbytes)
        return t

    @property
    def dev(self) -> CUDA:
        return self.buf.dev

    @property
    def device(self) -> str:
        return self.buf.dev.device

    @property
    def ptr(self) -> int:
        return self.buf.ptr

    @property
    def nbytes(self) -> int:
        return self.buf.nbytes

    def numel(self) -> int:
        return int(math.prod(self.shape))

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        shape = list(shape)
        if -1 in shape:
            i = shape.index(-1)
            shape[i] = self.numel() // int(-math.prod(shape))
        assert math.prod(shape) == self.numel(), f"cannot reshape {self.shape} to {shape}"
        return Tensor(self.buf, shape=shape)

    def view_rows(self, start: int, stop: int) -> "Tensor":
        """shrink on axis 0 of a contiguous tensor (an `_offset` sub-buffer, no copy)."""
        row = self.numel() // self.shape[0]
        b = self.buf.view((stop - start) * row, self.dtype, start * row * _DTYPE_SIZE[self.dtype])
        return Tensor(b, shape=(stop - start,) + tuple(self.shape[1:]))

    def assign(self, arr: np.ndarray) -> "Tensor":
        self.buf.copyin(np.asarray(arr, dtype=_NP[self.dtype]).reshape(self.shape))
        return self

    def realize(self) -> "Tensor":
        return self

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, _NP[self.dtype])
        self.buf.copyout(out)
        return out

    def item(self):
        assert self.numel() == 1
        return self.numpy().reshape(-1)[0].item()

    def tolist(self):
        return self.numpy().tolist()

    def to(self, device: str | CUDA) -> "Tensor":
        dst = device if isinstance(device, CUDA) else Device[device]
        if dst is self.dev:
            return self
        out = Tensor.empty(self.shape, self.dtype, dst)
        dst.allocator._transfer(out.ptr, self.ptr, self.nbytes, self.dev, dst)
        return out


class CompileError(RuntimeError):
    """jsgrad/runtime/allocator.ts:121."""


class CUDACompiler:
    """Compiler (jsgrad/runtime/allocator.ts:123-139): ``compile(src) -> bytes`` (a cubin) with a cache keyed by the
    source, as ``compile_cached`` keeps one on disk.  Needs no device."""

    def __init__(self, arch: str = "sm_100a"):
        self.arch = arch
        self._cache: dict[str, bytes] = {}

    def compile(self, src: str) -> bytes:
        ffi.load()
        image, size = C.c_void_p(), C.c_uint64(0)
        try:
            ffi.call("jg_cuda_compile", src.encode(), self.arch.encode(), C.byref(image), C.byref(size))
        except ffi.JgError as e:
            if e.status == ffi.JG_EINVAL:
                raise CompileError(str(e)) from None
            raise
        try:
            return C.string_at(image, size.value)
        finally:
            ffi.call("jg_cuda_image_free", image)

    def compile_cached(self, src: str) -> bytes:
        lib = self._cache.get(src)
        if lib is None:
            lib = self._cache[src] = self.compile(src)
        return lib


class CUDAProgram:
    """Program (jsgrad/runtime/allocator.ts:99-107; ops_clang.ts:30-54): ``CUDAProgram(dev, name, lib)`` loads the
    kernel ``name`` of the cubin ``lib``; calling it launches ``global_size`` blocks of ``local_size`` threads with
    the buffers as device pointers followed by ``vals`` as 32-bit ints.  ``wait=True`` returns the elapsed device
    time in seconds."""

    def __init__(self, dev: CUDA, name: str, lib: bytes):
        if not lib:
            raise ValueError("Lib is empty")  # ops_clang.ts:34
        if not name:
            raise ValueError("Name can't be undefined")  # ops_clang.ts:35
        self.dev, self.name, self.lib = dev, name, lib
        self.handle: C.c_void_p | None = None
        h = C.c_void_p()
        ffi.call("jg_program_load", dev.handle, name.encode(), lib, len(lib), C.byref(h))
        self.handle = h

    def __call__(self, *bufs, global_size: Sequence[int] | None = None, local_size: Sequence[int] | None = None,
                 vals: Sequence[int] = (), wait: bool = False) -> float | None:
        ptrs = [b if isinstance(b, int) else b.ptr for b in bufs]
        barr = (C.c_uint64 * max(len(ptrs), 1))(*ptrs)
        varr = (C.c_int32 * max(len(vals), 1))(*[int(v) for v in vals])
        three = lambda v: None if v is None else (C.c_uint32 * 3)(*(list(v) + [1, 1, 1])[:3])
        if wait:
            self.dev.timer_start()
        ffi.call("jg_program_call", self.handle, barr, len(ptrs), varr, len(vals), three(global_size), three(local_size))
        return self.dev.timer_stop() if wait else None

    def close(self) -> None:
        if self.handle is not None:
            ffi.call("jg_program_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            if self.dev.handle is not None:
                self.close()
        except Exception:
            pass


class CUDAGraph:
    """A captured kernel list replayed with one launch (GraphRunner, jsgrad/engine/jit.ts:71-141).  Values that
    vary between replays are device-resident (tokens, positions), so nothing is patched at launch."""

    def __init__(self, dev: CUDA):
        self.dev = dev
        self.handle: C.c_void_p | None = None

    def __enter__(self) -> "CUDAGraph":
        self.dev.call("jg_graph_begin")
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        h = C.c_void_p()
        if exc_type is not None:
            try:  # leave capture mode; the partial graph is discarded
                ffi.call("jg_graph_end", self.dev.handle, C.byref(h))
                ffi.call("jg_graph_destroy", h)
            except ffi.JgError:
                pass
            return False
        ffi.call("jg_graph_end", self.dev.handle, C.byref(h))
        self.handle = h
        return False

    def launch(self) -> None:
        ffi.call("jg_graph_launch", self.dev.handle, self.handle)

    def __del__(self):
        try:
            if self.handle is not None and self.dev.handle is not None:
                ffi.call("jg_graph_destroy", self.handle)
        except Exception:
            pass
