"""CPU-side checks of the boundary: the shared library loads, exports every symbol the header declares, the ctypes
table covers the header one to one, and the device path fails loudly (no fallback) where there is no GPU."""
import ctypes
import os
import re

import pytest

from denograd_b200 import ffi
from tests.util import ROOT

HEADER = os.path.join(ROOT, "include", "jsgrad_cuda.h")


def header_functions() -> dict[str, int]:
    """name -> number of parameters, parsed from the declarations in the header."""
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int|const char\*)\s+(jg_\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        params = m.group(2).strip()
        out[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    return out


def test_header_declares_expected_surface():
    fns = header_functions()
    for must in ("jg_device_open", "jg_alloc", "jg_free", "jg_copyin", "jg_copyout", "jg_transfer", "jg_graph_launch",
                 "jg_linear", "jg_norm_linear", "jg_norm_swiglu", "jg_rmsnorm", "jg_embed", "jg_rope_kvwrite",
                 "jg_attn_decode", "jg_norm_logits_argmax", "jg_argmax", "jg_freqs_cis", "jg_last_error"):
        assert must in fns, must


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(ffi.LIB_PATH)
    for name in header_functions():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_table_matches_header():
    fns = header_functions()
    declared = {k: v for k, v in fns.items() if k != "jg_last_error"}
    assert set(declared) == set(ffi.SIGNATURES), set(declared) ^ set(ffi.SIGNATURES)
    for name, n in declared.items():
        assert len(ffi.SIGNATURES[name]) == n, f"{name}: header has {n} parameters, ctypes table {len(ffi.SIGNATURES[name])}"
    ffi.load()  # sets argtypes on every symbol; raises if one is missing


def test_only_jg_symbols_are_exported():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", ffi.LIB_PATH], capture_output=True, text=True).stdout
    names = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert names and all(n.startswith("jg_") for n in names), [n for n in names if not n.startswith("jg_")][:5]


def _no_gpu() -> bool:
    n = ctypes.c_int32(0)
    return ffi.load().jg_device_count(ctypes.byref(n)) != 0 or n.value == 0


@pytest.mark.skipif(not _no_gpu(), reason="a CUDA device is present")
def test_no_device_fails_loudly():
    """Without a GPU the device cannot be opened and nothing silently falls back to the CPU."""
    from denograd_b200.device import CUDA
    with pytest.raises(ffi.JgError) as e:
        CUDA("CUDA").init()
    assert e.value.status in (ffi.JG_EIO, ffi.JG_EINVAL)
    assert str(e.value)


def test_device_names():
    from denograd_b200.device import Device
    assert Device.canonicalize("cuda") == "CUDA" and Device.canonicalize("CUDA:0") == "CUDA"
    assert Device.canonicalize("CUDA:3") == "CUDA:3"
    with pytest.raises(ValueError):
        Device.canonicalize("CLANG")


def test_typescript_symbol_table_matches_header():
    """The Deno.dlopen table of ts/ops_cuda.ts lists every function of the header with the same parameter count."""
    src = open(os.path.join(ROOT, "denograd_b200", "ts", "ops_cuda.ts")).read()
    start = src.index("export const SYMBOLS = {")
    body = src[start:src.index("\n} as const", start)]
    ts = {}
    for m in re.finditer(r"(jg_\w+):\s*fn\(\[([^\]]*)\]", body):
        ts[m.group(1)] = len([p for p in m.group(2).split(",") if p.strip()])
    assert "jg_last_error" in body
    declared = {k: v for k, v in header_functions().items() if k != "jg_last_error"}
    assert set(ts) == set(declared), set(ts) ^ set(declared)
    for name, n in declared.items():
        assert ts[name] == n, f"{name}: header has {n} parameters, ops_cuda.ts {ts[name]}"
