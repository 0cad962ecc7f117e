"""The TypeScript half of the kernel-substitution seam, pinned without a JS runtime.

denograd_b200/ts/llama_cuda.ts maps every Llama block step onto the library's entry points; no Deno exists here to run
it.  What can be checked mechanically is checked: (1) the `cu(dev, '<entry>', ...)` lines of the TypeScript source equal
ts/call_plan.json; (2) the Python twin (denograd_b200/llama.py), run against a recording stand-in for the library,
issues exactly the plan's entry points with exactly the plan's arguments — each TypeScript argument expression is
evaluated against the Python objects and compared with the recorded value; (3) the three symbol tables (header, ctypes,
Deno.dlopen) agree in parameter *types*, not only in count; (4) every entry point the TypeScript layers call exists in
the Deno symbol table with that many parameters."""
import ctypes as C
import importlib.util
import json
import os
import re

import numpy as np
import pytest

from denograd_b200 import ffi
from tests.fake_ffi import recording
from tests.golden.gen_golden import TINY
from tests.test_abi import HEADER
from tests.util import ROOT

TS_DIR = os.path.join(ROOT, "denograd_b200", "ts")


def _gen():
    spec = importlib.util.spec_from_file_location("gen_call_plan", os.path.join(TS_DIR, "gen_call_plan.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def plan() -> dict:
    return json.load(open(os.path.join(TS_DIR, "call_plan.json")))


def test_typescript_source_equals_the_committed_plan():
    assert _gen().parse_ts(os.path.join(TS_DIR, "llama_cuda.ts")) == plan()


# ---- evaluation of a TypeScript argument expression against the Python twin's objects
ALIAS = {"wqkv": "_wqkv", "layer": "_layer", "vocab_size": "vocab_local"}


def resolve(expr: str, roots: dict):
    if re.fullmatch(r"-?\d+", expr):
        return int(expr)
    parts = expr.split(".")
    obj = roots[parts[0]]
    for p in parts[1:]:
        obj = getattr(obj, ALIAS.get(p, p))
    if hasattr(obj, "weight"):          # a layer passed whole: its weight's address (`cu` takes `.ptr`)
        obj = obj.weight
    if hasattr(obj, "ptr") and not isinstance(obj, (int, float)):
        return obj.ptr
    if isinstance(obj, C.c_void_p):
        return obj.value
    return obj


def same(a, b) -> bool:
    if isinstance(a, float) or isinstance(b, float):
        return abs(float(a) - float(b)) <= 1e-12 * max(1.0, abs(float(b)))
    return a == b


def check_calls(recorded: list[tuple], expected: list[dict], roots: dict, what: str):
    assert [c[0] for c in recorded] == [e["entry"] for e in expected], (what, [c[0] for c in recorded], [e["entry"] for e in expected])
    for rec, exp in zip(recorded, expected):
        want = [resolve(x, roots) for x in exp["args"]]
        got = list(rec[1:])
        assert len(got) == len(want), (what, exp["entry"], got, exp["args"])
        for g, w, x in zip(got, want, exp["args"]):
            assert same(g, w), f"{what}: {exp['entry']} argument `{x}`: Python passes {g}, the TypeScript expression gives {w}"


@pytest.mark.parametrize("quant,B,mode", [("float16", 1, "fused"), ("float16", 2, "fused"), ("float16", 4, "rows"), ("int8", 1, "fused"), ("int8", 3, "rows")])
def test_python_twin_issues_the_planned_decode_step(quant, B, mode, monkeypatch):
    P = plan()
    monkeypatch.setenv("JG_STEP_KERNEL", "0")  # the launch-per-op step (the single-kernel one has its own test below)
    with recording() as rec:
        from denograd_b200.llama3 import Llama3
        args = dict(TINY, dim=512) if quant == "int8" else TINY  # the int8 one-row kernel wants dim % 512 == 0
        llm = Llama3(size="1B", args=args, quantize=quant, max_context=64, max_batch=8, tied_output=False, temperature=0)
        m = llm.model
        ws = m._workspace(B)
        n0 = len(rec.calls)
        m._step(ws)
        got = rec.kernels(n0)
        L = len(m.layers)
        per = len(P["decode_step_fused" if mode == "fused" else "decode_step_rows"])
        top = {"ws": ws, "this": m, "B": B}
        check_calls(got[:1], P["decode_step"][:1], top, "embedding")
        for l, layer in enumerate(m.layers):
            roots = {"ws": ws, "this": layer, "a": layer.attention, "f": layer.feed_forward, "B": B, "dim": m.dim, "kv": m._kv,
                     "freqs_cis": m.freqs_cis, "freqs_rows": m.freqs_cis.shape[0]}
            check_calls(got[1 + l * per:1 + (l + 1) * per], P["decode_step_fused" if mode == "fused" else "decode_step_rows"], roots, f"layer {l}")
        tail = got[1 + L * per:]
        want_tail = [P["decode_step"][1], P["decode_step"][4]] if mode == "fused" else P["decode_step"][2:5]
        check_calls(tail, want_tail, top, "output layer")
        del llm, m, ws


@pytest.mark.parametrize("B", [1, 2])
def test_python_twin_issues_the_single_kernel_step(B):
    """fp16 weights, 1-2 rows: the whole step is one jg_step_run on the plan's handle, same arguments on both sides."""
    P = plan()
    with recording() as rec:
        from denograd_b200.llama3 import Llama3
        llm = Llama3(size="1B", args=TINY, max_context=64, max_batch=2, tied_output=False, temperature=0)
        m = llm.model
        ws = m._workspace(B)
        n0 = len(rec.calls)
        m._step(ws)
        got = rec.kernels(n0)
        created = [c for c in rec.calls[n0:] if c[0] == "jg_step_create"]
        assert len(created) == 1 and [c[0] for c in got] == ["jg_step_run"], [c[0] for c in got]
        check_calls(got[:1], P["decode_step_single"], {"ws": ws, "this": m, "B": B}, "single-kernel step")
        m._step(ws)  # the plan is made once
        assert sum(1 for c in rec.calls[n0:] if c[0] == "jg_step_create") == 1
        del llm, m, ws


def test_python_twin_issues_the_planned_prefill_chunk():
    P = plan()
    with recording() as rec:
        from denograd_b200.llama3 import Llama3
        llm = Llama3(size="1B", args=TINY, max_context=64, max_batch=2, tied_output=False, temperature=0)
        m = llm.model
        toks = np.arange(2 * 12, dtype=np.int32).reshape(2, 12) % TINY["vocab_size"]
        n0 = len(rec.calls)
        m._forward_rows(toks, 0, last=True)
        got = rec.kernels(n0)
        R, bsz, sc = 24, 2, 12
        ws, wsb = m._workspace(R, rows=True), m._workspace(bsz)
        per = len(P["prefill_chunk"])
        check_calls(got[:1], P["forward"][:1], {"ws": ws, "this": m, "R": R}, "embedding")
        for l, layer in enumerate(m.layers):
            roots = {"ws": ws, "this": layer, "a": layer.attention, "f": layer.feed_forward, "R": R, "dim": m.dim, "kv": m._kv,
                     "freqs_cis": m.freqs_cis, "freqs_rows": m.freqs_cis.shape[0], "batch": bsz, "positions": sc}
            check_calls(got[1 + l * per:1 + (l + 1) * per], P["prefill_chunk"], roots, f"layer {l}")

        class P_:  # the rows of the last position inside the chunk's buffers
            def __init__(self, ptr): self.ptr = ptr
        tail_roots = {"wsb": wsb, "this": m, "bsz": bsz, "h_last": P_(ws.h.ptr + 2 * m.dim * (R - bsz)), "xn_last": P_(ws.xn.ptr + 2 * m.dim * (R - bsz))}
        check_calls(got[1 + len(m.layers) * per:], P["forward"][1:], tail_roots, "output layer of the chunk")
        del llm, m, ws, wsb


# ---- parameter types across the three tables
C_TO_KIND = {"uint64_t": "u64", "int32_t": "i32", "int64_t": "i64", "float": "f32", "double": "f64", "size_t": "usize"}
CTYPES_KIND = {C.c_uint64: "u64", C.c_int32: "i32", C.c_int64: "i64", C.c_float: "f32", C.c_double: "f64", C.c_size_t: "usize",
               C.c_void_p: "ptr", C.c_char_p: "ptr"}


def header_param_kinds() -> dict[str, list[str]]:
    src = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    out = {}
    for m in re.finditer(r"\bint\s+(jg_\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        params = m.group(2).strip()
        kinds = []
        if params not in ("", "void"):
            for p in params.split(","):
                p = " ".join(p.split())
                kinds.append("ptr" if "*" in p else C_TO_KIND[p.replace("const ", "").rsplit(" ", 1)[0]])
        out[m.group(1)] = kinds
    return out


def test_parameter_types_agree_between_header_ctypes_and_typescript():
    hdr = header_param_kinds()
    ts_src = open(os.path.join(TS_DIR, "ops_cuda.ts")).read()
    body = ts_src[ts_src.index("export const SYMBOLS = {"):]
    body = body[:body.index("\n} as const")]
    ts_kind = {"u64": "u64", "i32": "i32", "f32": "f32", "f64": "f64", "ptr": "ptr", "buf": "ptr", "usize": "usize", "'i64'": "i64"}
    for name, kinds in hdr.items():
        py = []
        for t in ffi.SIGNATURES[name]:
            py.append(CTYPES_KIND.get(t, "ptr"))  # POINTER(...) types are pointers
        # size_t and uint64_t are the same 8-byte integer on this ABI: the tables may name either
        norm = lambda ks: ["u64" if k == "usize" else k for k in ks]
        assert norm(py) == norm(kinds), f"{name}: ctypes {py} vs header {kinds}"
        m = re.search(rf"\b{name}:\s*fn\(\[([^\]]*)\]", body)
        assert m, name
        ts = [ts_kind[p.strip()] for p in m.group(1).split(",") if p.strip()]
        assert norm(ts) == norm(kinds), f"{name}: ops_cuda.ts {ts} vs header {kinds}"


def test_every_entry_point_the_typescript_layers_call_is_bound():
    ts_src = open(os.path.join(TS_DIR, "ops_cuda.ts")).read()
    body = ts_src[ts_src.index("export const SYMBOLS = {"):]
    body = body[:body.index("\n} as const")]
    arity = {m.group(1): len([p for p in m.group(2).split(",") if p.strip()]) for m in re.finditer(r"(jg_\w+):\s*fn\(\[([^\]]*)\]", body)}
    P = plan()
    for method, calls in P.items():
        for c in calls:
            assert c["entry"] in arity, (method, c["entry"])
            assert arity[c["entry"]] == len(c["args"]) + 1, (method, c["entry"], "the device handle is the first C argument")
    assert "extends GraphRunner" in ts_src and "CUDAProgram.bind(this)" in ts_src and "this.graph =" in ts_src
