"""A stand-in for the C library that records calls instead of launching kernels, so that the host-side call sequences of
denograd_b200 can be checked on a machine without a GPU.  It implements just enough of the allocation / handle entry
points to let the model objects be built: device addresses are handed out from a counter, handles are small integers,
page-locked host memory is ordinary memory.  Nothing is computed."""
from __future__ import annotations

import contextlib
import ctypes as C

from denograd_b200 import device as D
from denograd_b200 import ffi


class Recorder:
    def __init__(self):
        self.calls: list[tuple] = []
        self._next_ptr = 0x10000000
        self._next_handle = 0x1000
        self._host: list = []

    @staticmethod
    def _plain(a):
        if isinstance(a, (C.c_void_p, C.c_uint64, C.c_int32, C.c_int64)):
            return a.value
        if isinstance(a, (bytes, C.Array)) or hasattr(a, "_obj"):  # byref(...) and buffers: not part of a call's identity
            return "<ref>"
        return a

    def call(self, name: str, *args) -> None:
        if name == "jg_device_open":
            args[1]._obj.value = self._handle()
        elif name == "jg_device_props":
            p = args[1]._obj
            p.sm_count, p.cc_major, p.max_smem_per_block = 148, 10, 232448
        elif name == "jg_alloc":
            args[2]._obj.value = self._next_ptr
            self._next_ptr += (int(args[1]) + 255) // 256 * 256
        elif name in ("jg_kvcache_create", "jg_graph_end", "jg_step_create"):
            args[-1]._obj.value = self._handle()
        elif name == "jg_host_alloc":
            buf = C.create_string_buffer(int(args[0]))
            self._host.append(buf)
            args[1]._obj.value = C.addressof(buf)
        elif name == "jg_launch_count":
            args[1]._obj.value = len(self.calls)
        elif name == "jg_kvcache_bytes":
            args[1]._obj.value = 0
        self.calls.append((name,) + tuple(self._plain(a) for a in args))

    def _handle(self) -> int:
        self._next_handle += 0x10
        return self._next_handle

    def kernels(self, since: int = 0) -> list[tuple]:
        """Recorded compute calls (everything but allocation, copies and bookkeeping), device handle stripped."""
        skip = {"jg_alloc", "jg_free", "jg_copyin", "jg_copyout", "jg_memset", "jg_host_alloc", "jg_host_free", "jg_device_open",
                "jg_device_props", "jg_device_sync", "jg_launch_count", "jg_kvcache_create", "jg_kvcache_destroy",
                "jg_kvcache_bytes", "jg_copyin_async", "jg_copyout_async", "jg_copy", "jg_freqs_cis", "jg_step_create",
                "jg_step_destroy"}
        return [(c[0],) + c[2:] for c in self.calls[since:] if c[0] not in skip]


@contextlib.contextmanager
def recording():
    """Route every ffi.call to a Recorder and give `Device[...]` fresh device objects for the duration."""
    rec = Recorder()
    saved_call, saved_load, saved_opened = ffi.call, ffi.load, dict(D.Device._opened)
    ffi.call = rec.call
    ffi.load = lambda: None
    D.Device._opened.clear()
    try:
        yield rec
    finally:
        for d in D.Device._opened.values():  # objects that outlive the block must not hand fake handles to the real library
            d.handle = None
        ffi.call, ffi.load = saved_call, saved_load
        D.Device._opened.clear()
        D.Device._opened.update(saved_opened)
