"""Benchmark of the Llama-3 greedy-decode hot path on the CUDA device (and of the CPU reference arm).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                  [--model 8B] [--quant float16|int8] [--batch B] [--prompt P]

A step is one decode step (one new token per batch row) of the whole model.  Default workload: Llama-3.1-8B
architecture, fp16 weights ~N(0, 0.02) (seeded, generated on the device), batch 1, 512-token seeded prompt already
in the KV cache, greedy decoding.  One JSON line is printed by rank 0:

  parity     before anything is timed: small and full-width reduced-depth models run through the very objects the
             timed legs use (the tensor-parallel communicator included) and are compared with the CPU checker
             (oracle/, used here only as the checker); a mismatch ends the run with a non-zero exit code;
  value      decode tokens/s with everything resident in HBM: the captured step replays back to back and feeds its own
             token back on the device (timed with CUDA events on the launching stream); exactly K steps, after which
             the region is repeated for `repeats` (median / min / max);
  e2e        the same metric through the public per-token API: token ids and positions are copied up from page-locked
             host memory, the step runs, the chosen ids are read back — every step, as the reference's chat loop does;
  roofline   the dominant kernel (the weight-streaming matrix-vector kernel, timed alone on the gate/up projection
             of every layer in turn) against the measured HBM copy bandwidth; `step` carries the same figure for the
             whole decode step (all weights + KV read once per step);
  extra      further legs of the same metric family, each with its own fraction of its roofline: prompt processing,
             batch-32 decode at a 512- and a 4096-token context, int8 weights (batch 1 / 8 decode at a 2048-token
             context, 2048-token prompt), the 3B and 1B architectures;
  cpu_baseline  the CPU restatement of the reference's CLANG path (oracle/), timed on this host's cores on a bounded
             sample: full-width 1-, 4- and 8-layer slices with 512 positions in the cache, extrapolated in depth.

`--impl reference` times that CPU restatement as the reference arm (the reference itself needs a JS runtime and
clang, neither of which exists here).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_second"
UNIT = "tok/s"


def measured_peaks() -> dict:
    """Roofline denominators: the driver-measured copy bandwidth and bf16 GEMM rates if present, else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return {"hbm_gbs": float(j["hbm_gbs"]), "tflops": float(j["bf16_tflops"]), "kind": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops": 1590.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self) -> int:
        return len(self.rows)

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()  # the exact child we started
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
            self.t.join(timeout=2)

    def summary(self, lo: int = 0, hi: int | None = None) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows[lo:hi]:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ workload sizes
LAYERS_OVERRIDE = 0


def arch(model: str):
    from denograd_b200.llama3 import MODEL_PARAMS
    p = dict(MODEL_PARAMS[model]["args"])
    if LAYERS_OVERRIDE:
        p["n_layers"] = LAYERS_OVERRIDE
    return p, MODEL_PARAMS[model]["tied"]


def layer_params(p: dict) -> int:
    d, hd = p["dim"], p["dim"] // p["n_heads"]
    kv, f = p["n_kv_heads"] * hd, p["hidden_dim"]
    return 2 * d * d + 2 * kv * d + 3 * f * d


def weight_bytes(p: dict, tied: bool, int8: bool) -> int:
    """Bytes of weights one decode step streams: every projection once, the output matrix once (the embedding
    gather touches one row per token)."""
    d, hd = p["dim"], p["dim"] // p["n_heads"]
    kv, f, V, L = p["n_kv_heads"] * hd, p["hidden_dim"], p["vocab_size"], p["n_layers"]
    params = L * layer_params(p) + V * d
    rows = L * (2 * d + 2 * kv + 2 * f + d) + V  # scale entries (one fp16 per output row) for int8
    return params * (1 if int8 else 2) + (rows * 2 if int8 else 0) + L * 2 * d * 2 + d * 2  # + norm weights


def kv_bytes_per_token(p: dict) -> int:
    hd = p["dim"] // p["n_heads"]
    return 2 * p["n_layers"] * p["n_kv_heads"] * hd * 2


def prefill_flops(p: dict, B: int, S: int) -> float:
    """Algorithmic flops of one multi-position forward over B sequences of S new tokens from an empty cache: every
    layer's projections on all B*S rows, the output matrix on the last row of each sequence only, causal attention
    (q.k and p.v, half of the S x S square)."""
    d, hd = p["dim"], p["dim"] // p["n_heads"]
    return (2.0 * B * S * p["n_layers"] * layer_params(p) + 2.0 * B * p["vocab_size"] * d
            + 4.0 * B * p["n_layers"] * p["n_heads"] * hd * S * S / 2.0)


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(model: str, int8: bool, steps: int, context: int = 512, with_single_thread: bool = True) -> dict:
    """Times the CPU restatement (oracle/) on full-width 1-, 4- and 8-layer slices of `model`, batch 1, with `context`
    positions already in the cache, and extrapolates the per-token time of the full depth from the 1- and 4-layer
    points: t(L) = t_head + L * t_layer; the 8-layer point checks the line.  The thread count is set explicitly to
    the host's cores (a launcher's OMP_NUM_THREADS is not inherited)."""
    from oracle import oracle as O  # the checker, used here only as the timed CPU baseline
    from tests.util import build_oracle
    from denograd_b200 import synth
    p, tied = arch(model)
    cores = os.cpu_count() or 1
    steps = max(3, min(steps, 16))
    rng = np.random.default_rng(1)

    def time_slice(L: int, threads: int, n: int) -> float:
        O.set_threads(cores)  # the seeded tensors are generated on all cores whatever the timed thread count is
        q = dict(p); q["n_layers"] = L
        m = build_oracle(q, max_context=context + n + 8, max_batch=1, int8=int8, tied=tied)
        O.set_threads(threads)
        cache = m.cache()  # stand-in K/V rows for the cached positions: the cost of attention depends on their number only
        cache[:, :, :, :context] = (rng.standard_normal(cache[:, :, :, :context].shape) * 0.5).astype(np.float16)
        toks = synth.prompt_tokens(n + 1, p["vocab_size"])
        m.forward(toks[:, 0:1], context)  # warm-up (page faults, caches)
        t0 = time.perf_counter()
        for i in range(n):
            m.forward(toks[:, i + 1:i + 2], context + 1 + i)
        dt = (time.perf_counter() - t0) / n
        m.close()
        return dt

    times = {L: time_slice(L, cores, steps) for L in (1, 4, 8)}
    # least-squares line through the three points; the 8-layer point against the line through the other two is the check
    xs, ys = np.array([1.0, 4.0, 8.0]), np.array([times[1], times[4], times[8]])
    t_layer, t_head = np.polyfit(xs, ys, 1)
    t_layer, t_head = max(float(t_layer), 1e-9), max(float(t_head), 0.0)
    t_full = t_head + p["n_layers"] * t_layer
    tl2 = (times[4] - times[1]) / 3.0
    pred8 = (times[1] - tl2) + 8 * tl2
    out = {"value": 1.0 / t_full, "unit": UNIT, "cores": cores, "kind": "port", "estimate": True,
           "sample": (f"{model} architecture, batch 1, {context} positions in the cache: {steps} greedy steps each on full-width "
                      f"1-, 4- and 8-layer slices (embedding + layers + final norm + {p['vocab_size']}-row output); per-token "
                      f"time extrapolated to {p['n_layers']} layers as t_head + L*t_layer (least-squares line through the three points) "
                      f"(t_head {t_head * 1e3:.1f} ms, t_layer {t_layer * 1e3:.1f} ms); OpenMP over output rows on "
                      f"{cores} threads, set explicitly (the reference's generated C itself is single-threaded)"),
           "ms_per_token_est": t_full * 1e3,
           "linearity_check": {"layers": 8, "measured_ms": times[8] * 1e3, "predicted_from_1_and_4_ms": pred8 * 1e3,
                               "rel_err": abs(times[8] - pred8) / times[8]}}
    if with_single_thread:
        n1 = 2
        t1 = {L: time_slice(L, 1, n1) for L in (1, 2)}
        tl1 = max(t1[2] - t1[1], 1e-9)
        th1 = max(t1[1] - tl1, 0.0)
        out["single_thread"] = {"value": 1.0 / (th1 + p["n_layers"] * tl1), "unit": UNIT, "cores": 1, "estimate": True,
                                "sample": f"the same on 1 thread (the reference's real shape): {n1} steps each on 1- and 2-layer slices"}
        O.set_threads(cores)
    return out


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    int8 = args.quant == "int8"
    cb = cpu_sample(args.model, int8, args.steps, context=args.prompt)
    p, tied = arch(args.model)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_token_est"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 weights, f32 accumulate", "data": "synthetic",
            "value_is": "estimate: per-token time of the full depth extrapolated from timed 1-, 4- and 8-layer slices (see cpu_baseline.sample)",
            "config": workload_config(args, p), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(args, p) -> dict:
    return {"workload": (f"Llama-3.1-{args.model} architecture greedy decode, {args.quant} weights, batch {args.batch}, "
                         f"{args.prompt}-token seeded prompt in the KV cache"),
            "batch": args.batch, "prompt_tokens": args.prompt, "weights": args.quant, "layers": p["n_layers"],
            "l2": "inputs larger than L2: every step streams all weights (GBs) once, no flush needed",
            "parallelism": f"tp{args.gpus}" + ("" if args.gpus == 1 else
                            ": heads / FFN width / vocabulary sharded; fp32 all-reduce after wo and w2 over NVLink peer memory: "
                            "pushed by the row-parallel projection and summed in the next projection's prologue (1-2 rows), "
                            "one-shot or two-shot exchange kernels (more rows), NCCL for prompt chunks")}


# ------------------------------------------------------------------------------------------------ GPU arm
class Rig:
    """Process-wide plumbing of one rank: device, (optional) torch.distributed group and tensor-parallel handle."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.dist = None
        self.tp = None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        from denograd_b200.device import Device
        self.dev_name = "CUDA" if self.local_rank == 0 else f"CUDA:{self.local_rank}"
        self.dev = Device[self.dev_name]
        if self.world > 1:
            # tensor parallel over the ranks: rank 0 makes the NCCL id, torch.distributed carries it to the others
            from denograd_b200.multi import TensorParallel, exchange_via_torch
            box = [TensorParallel.unique_id() if self.rank == 0 else None]
            self.dist.broadcast_object_list(box, src=0)
            self.tp = TensorParallel(self.dev, self.rank, self.world, box[0])
            if os.environ.get("JG_TP_PEER", "1") != "0":
                self.tp.open_peers(exchange_via_torch)  # exchanges as kernels over NVLink peer memory

    def barrier(self):
        self.dev.synchronize()
        if self.dist is not None:
            self.dist.barrier()

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{self.local_rank}")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def same_on_all_ranks(self, arr: np.ndarray) -> bool:
        if self.dist is None:
            return True
        out = [None] * self.world
        self.dist.all_gather_object(out, np.asarray(arr).tobytes())
        return all(o == out[0] for o in out)

    def llama(self, model: str, quant: str, max_ctx: int, max_batch: int, n_layers=None, args=None, tied=None):
        from denograd_b200.llama3 import Llama3
        return Llama3(size=model, quantize=quant, max_context=max_ctx, max_batch=max_batch, device=self.dev_name, temperature=0.0,
                      n_layers=n_layers, tp=self.tp, args=args or {}, tied_output=tied).load_synthetic()

    def release(self):
        gc.collect()
        self.dev.synchronize()
        self.dev.allocator.free_cache()


# Small architecture whose heads, kv heads, FFN width and vocabulary divide by 8, for the parity cases at every N.
SMALL8 = {"dim": 512, "n_heads": 8, "n_kv_heads": 8, "n_layers": 2, "norm_eps": 1e-5, "rope_theta": 500000,
          "vocab_size": 2048, "hidden_dim": 1024}


def parity_checks(rig: Rig) -> dict:
    """Correctness of what is about to be timed, at this world size: greedy ids and last logits of (a) a small model at
    batch 2 (1-2 rows: split exchange under tensor parallelism), (b) the same at batch 5 (one-shot exchange kernel),
    (c) a 2-layer full-width 8B slice at batch 1 through prefill-by-token + decode and (d) the same slice over one
    64-row prompt chunk (two-shot exchange / tensor-core projections), each against the CPU checker on rank 0.  Ids are
    compared up to the first step whose checker margin is below 3 fp16 ulp (a near-tie may legitimately flip)."""
    from denograd_b200 import synth
    from denograd_b200.llama3 import MODEL_PARAMS
    from oracle import oracle as O  # checker only; never inside a timed region
    from tests.util import build_oracle, oracle_greedy
    O.set_threads(os.cpu_count() or 1)
    cases, ids_equal, max_dlogit, tie_steps, failures = 0, True, 0.0, 0, []
    checkers: dict = {}  # one checker model per (architecture, batch): its seeded weights take seconds to generate

    def run_case(name, size, arch_args, tied, batch, prompt_len, n_new, chunk):
        nonlocal cases, ids_equal, max_dlogit, tie_steps
        p = dict(MODEL_PARAMS[size]["args"]); p.update(arch_args)
        prompt = synth.prompt_tokens(prompt_len, p["vocab_size"], batch=batch, seed=31)
        llm = rig.llama(size, "float16", 128, batch, args=arch_args, tied=tied)
        if chunk:
            first = llm.prefill(prompt).numpy()
            ids = first.reshape(batch, 1)
        else:
            ids = llm.generate(prompt, n_new)
        logits = llm.model.last_logits(batch)  # this rank's vocabulary slice
        v0, vl = llm.model.vocab_offset, llm.model.vocab_local
        same = rig.same_on_all_ranks(ids)
        del llm
        rig.release()
        cases += 1
        if not same:
            ids_equal = False
            failures.append(f"{name}: ranks disagree on the ids")
        if rig.rank != 0:
            return
        ck = (size, tuple(sorted(arch_args.items())), tied, batch)
        if ck not in checkers:
            checkers[ck] = build_oracle(p, max_context=128, max_batch=batch, int8=False, tied=tied)
        m = checkers[ck]
        if chunk:
            ref_logits, ref_next = m.forward(prompt, 0)
            ref_ids, ref_all = ref_next.reshape(batch, 1), ref_logits[None]
            top2 = np.partition(ref_logits, -2, axis=1)[:, -2:]
            margins = (top2[:, 1] - top2[:, 0])[None]
        else:
            ref_ids, ref_all, margins = oracle_greedy(m, prompt, n_new)
        ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref_all.max(axis=2)), 1e-6))) - 10)
        safe = (margins / ulp) >= 3
        tie_steps += int((~safe).sum())
        full_match = True
        for b in range(batch):
            n = ids.shape[1] if safe[:, b].all() else int(np.argmin(safe[:, b]))
            if not (ids[b, :n] == ref_ids[b, :n]).all():
                ids_equal = False
                failures.append(f"{name}: row {b} ids {ids[b].tolist()} != checker {ref_ids[b].tolist()}")
            full_match &= bool((ids[b] == ref_ids[b]).all())
        if full_match:  # the last logits are comparable only on the same trajectory
            dl = float(np.abs(logits - ref_all[-1][:, v0:v0 + vl]).max())
            max_dlogit = max(max_dlogit, dl)
            if dl > 2e-2:
                failures.append(f"{name}: max |dlogit| {dl:.3e} exceeds 2e-2")

    run_case("small, batch 2", "1B", SMALL8, True, 2, 6, 6, False)
    run_case("small, batch 5", "1B", SMALL8, True, 5, 4, 4, False)
    run_case("8B 2-layer slice, batch 1", "8B", {"n_layers": 2}, False, 1, 4, 4, False)
    run_case("8B 2-layer slice, one 64-row chunk", "8B", {"n_layers": 2}, False, 1, 64, 1, True)
    for m in checkers.values():
        m.close()
    out = {"cases": cases, "ids_equal": bool(ids_equal and not failures), "max_dlogit": max_dlogit,
           "tie_sensitive_steps": tie_steps, "world": rig.world}
    if failures:
        out["failures"] = failures
    return out


def decode_leg(rig: Rig, llm, B: int, P: int, K: int, W: int, repeats: int, tied: bool, int8: bool, check_steps: int = 8) -> dict:
    """Prefill a seeded P-token prompt for B rows, then time K replayed decode steps `repeats` times (device loop, CUDA
    events, max over ranks).  Afterwards the same steps are redone through the per-token host API and through the
    device loop from the same state and their ids compared (and compared across ranks)."""
    from denograd_b200 import synth
    p = llm.params
    model, dev = llm.model, llm.model.dev
    prompt = synth.prompt_tokens(P, p["vocab_size"], batch=B, seed=synth.PROMPT_SEED)
    llm.reset()
    first = llm.prefill(prompt).numpy()
    pos0 = llm.start_pos
    model.decode_loop(first, pos0, W, collect=False)  # warm-up steps (also captures the step)
    times = []
    pos = pos0 + W
    launches0 = dev.launch_count()
    for _ in range(repeats):
        rig.barrier()
        dev.timer_start()
        model.decode_loop(first, pos, K, collect=False, resume=True)
        secs = dev.timer_stop()
        rig.barrier()
        times.append(rig.max_over_ranks(secs))
        pos += K
    launches = (dev.launch_count() - launches0) // repeats
    # ids: device loop against the per-token API from the same state (positions pos0.. are simply overwritten)
    loop_ids = model.decode_loop(first, pos0, check_steps)
    api = np.empty((B, check_steps), np.int32)
    tok = first
    for i in range(check_steps):
        tok = model.call_host(tok.reshape(B, 1), pos0 + i)
        api[:, i] = tok
    ok = bool((loop_ids == api).all()) and rig.same_on_all_ranks(api)
    if not ok:
        raise SystemExit(f"decode ids differ between the device loop and the per-token API (batch {B}): {loop_ids.tolist()} vs {api.tolist()}")
    med = statistics.median(times)
    t_mid = pos0 + W + (repeats * K) / 2.0  # mean cached length over the timed steps
    step_bytes = (weight_bytes(p, tied, int8) + B * t_mid * kv_bytes_per_token(p)) / rig.world + B * p["dim"] * 2  # per GPU
    peak = measured_peaks()["hbm_gbs"]
    return {"tok_s": B * K / med, "tok_s_min": B * K / max(times), "tok_s_max": B * K / min(times), "ms_per_step": med / K * 1e3,
            "batch": B, "steps": K, "repeats": repeats, "context": int(t_mid), "gpu_launches_per_region": int(launches),
            "bytes_per_step_per_gpu": step_bytes, "frac_of_hbm_roofline": step_bytes / (med / K) / 1e9 / peak,
            "ids_loop_equal_api": ok, "_secs": med, "_pos_end": pos, "_first": first, "_pos0": pos0}


def prefill_leg(rig: Rig, llm, B: int, P: int, int8: bool, reps: int = 3) -> dict:
    from denograd_b200 import synth
    p = llm.params
    dev = llm.model.dev
    prompt = synth.prompt_tokens(P, p["vocab_size"], batch=B, seed=synth.PROMPT_SEED)
    llm.reset(); llm.prefill(prompt); dev.synchronize()  # warm-up (kernels' attributes, workspaces)
    rig.barrier()
    dev.timer_start()
    for _ in range(reps):
        llm.reset()
        llm.prefill(prompt)
    pf = rig.max_over_ranks(dev.timer_stop()) / reps
    fl = prefill_flops(p, B, P) / rig.world
    tf = measured_peaks()["tflops"]
    return {"tok_s": B * P / pf, "ms": pf * 1e3, "prompt_tokens": P, "batch": B, "tflops_per_gpu": fl / pf / 1e12,
            "frac_of_measured_bf16_peak": fl / pf / 1e12 / tf,
            "flops": "layers on all rows + output matrix on the last row + causal attention",
            "how": ("Transformer.forward over the whole prompt in chunks of up to 2048 rows: tcgen05/TMA projections"
                    + (" over int8 weights" if int8 else "") + ", tensor-core causal attention")}


def run_gpu(args) -> None:
    rig = Rig()
    rank, world, dev = rig.rank, rig.world, rig.dev
    int8 = args.quant == "int8"
    p, tied = arch(args.model)
    B, P, K, W = args.batch, args.prompt, args.steps, args.warmup
    R = max(1, args.repeats)
    peaks = measured_peaks()
    peak = peaks["hbm_gbs"]

    parity = None
    if not args.no_parity:
        parity = parity_checks(rig)
        bad = [0 if parity["ids_equal"] else 1]
        if rig.dist is not None:
            rig.dist.broadcast_object_list(bad, src=0)
        if bad[0]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "parity": parity, "error": "parity check failed; nothing was timed"}))
            if rig.dist is not None:
                rig.dist.destroy_process_group()
            sys.exit(3)

    max_ctx = (P + (R + 1) * K + W + 64 + 63) // 64 * 64
    llm = rig.llama(args.model, args.quant, max_ctx, B, n_layers=p["n_layers"])
    model = llm.model
    with ClockSampler(rig.local_rank) as clocks:
        # ---- value: device-resident loop (graph replay, token fed back on the device)
        c0 = clocks.mark()
        main = decode_leg(rig, llm, B, P, K, W, R, tied, int8)
        c1 = clocks.mark()
        secs = main["_secs"]
        value = B * K / secs  # one model sharded over the ranks: the job's tokens are the batch's tokens

        # ---- e2e: public per-token API with host buffers (pinned H2D of ids + positions, D2H of the chosen ids)
        pos = main["_pos_end"]
        tok = model._workspace(B).next_tokens.numpy()
        for _ in range(W):
            tok = model.call_host(tok.reshape(B, 1), pos); pos += 1
        rig.barrier()
        dev.timer_start()
        for _ in range(K):
            tok = model.call_host(tok.reshape(B, 1), pos); pos += 1
        e2e_secs = rig.max_over_ranks(dev.timer_stop())
        rig.barrier()
        e2e_value = B * K / e2e_secs

        # ---- roofline of the dominant kernel, timed alone: gate/up projection (norm + two matrices + SwiGLU) of every
        #      layer in turn, so that consecutive launches never find their weights in L2
        ws = model._workspace(B)
        d, f = p["dim"], p["hidden_dim"] // world  # f: this rank's share of the FFN width
        from denograd_b200.llama import _norm_first
        big = _norm_first(B, int8)  # the projection takes pre-normalised rows and runs on the tensor cores

        def gateup(layer):
            ff = layer.feed_forward
            dev.call("jg_norm_swiglu", ws.ffn.ptr, (ws.xn if big else ws.h).ptr, 0 if big else layer.ffn_norm.weight.ptr,
                     layer.ffn_norm.eps, ff.w1.weight.ptr, ff.w1.scale_ptr, ff.w3.weight.ptr, ff.w3.scale_ptr, B, f, d)

        for layer in model.layers:
            gateup(layer)
        dev.synchronize()
        reps = max(1, 128 // len(model.layers))
        dev.timer_start()
        for _ in range(reps):
            for layer in model.layers:
                gateup(layer)
        k_secs = dev.timer_stop() / (reps * len(model.layers))
        k_bytes = 2 * f * d * (1 if int8 else 2) + (2 * f * 2 if int8 else 0) + B * d * 2 + d * 2 + B * f * 2
        k_gbs = k_bytes / k_secs / 1e9
        traffic = captured_traffic(args.model, args.quant, B, world)
        single = model._single_kernel_step(B) is not None  # the timed region is ONE launch of the persistent step kernel

        kernel_name = (("gemm_small_kernel (mma.sync, gate/up + SwiGLU instantiation)" if (int8 or B < 9) else
                        "gemm_tc_kernel (tcgen05, gate/up + SwiGLU instantiation)") if big else
                       "jg_matvec_kernel (norm + gate/up + SwiGLU instantiation)")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": secs / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 activations, f32 accumulate, " + ("i8 weights" if int8 else "f16 weights"), "data": "synthetic",
            "config": workload_config(args, p),
            "repeats": {"n": R, "steps_each": K, "tok_s_median": main["tok_s"], "tok_s_min": main["tok_s_min"], "tok_s_max": main["tok_s_max"]},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 4 * B,
                    "ms_per_step": e2e_secs / K * 1e3},
            "gpu_launches": int(main["gpu_launches_per_region"]),
            "parity": parity,
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": k_gbs,
                         "peak": peak, "peak_kind": peaks["kind"], "unit": "GB/s", "frac": k_gbs / peak, "traffic": traffic,
                         "bytes_per_launch": k_bytes, "us_per_launch": k_secs * 1e6,
                         "step": {"bytes_per_step": main["bytes_per_step_per_gpu"], "achieved": main["bytes_per_step_per_gpu"] / (secs / K) / 1e9,
                                  "frac": main["frac_of_hbm_roofline"],
                                  "hbm_roofline_tok_s": B * peak * 1e9 / main["bytes_per_step_per_gpu"], "per_gpu": True}},
        }
        if single:
            # the dominant (only) kernel of the timed region is the step kernel itself: one launch runs the K steps, its
            # algorithmic bytes are K steps' worth; the stand-alone gate/up projection stays beside it for comparison
            r = line["roofline"]
            step_bytes = main["bytes_per_step_per_gpu"]
            per_step = captured_traffic(args.model, args.quant, B, world, "dram_bytes_per_step", "/step")
            line["roofline"] = {
                "bound": "hbm", "kernel": "jg_step_kernel (the whole decode step as one persistent kernel; one launch = the region's steps)",
                "achieved": step_bytes / (secs / K) / 1e9, "peak": peak, "peak_kind": peaks["kind"], "unit": "GB/s",
                "frac": main["frac_of_hbm_roofline"], "traffic": per_step * K if per_step else None,
                "bytes_per_launch": step_bytes * K, "us_per_launch": secs * 1e6, "steps_per_launch": K,
                "step": r["step"],
                "standalone_gate_up": {k: r[k] for k in ("kernel", "achieved", "frac", "traffic", "bytes_per_launch", "us_per_launch")},
            }
        # ---- extra legs of the same metric family
        if not args.no_extra:
            extra = {}
            extra["prefill"] = prefill_leg(rig, llm, 1, P, int8)
            del model, ws, llm
            rig.release()
            extra.update(extra_legs(rig, args, R))
            line["extra"] = extra
        c2 = clocks.mark()
    line["clocks"] = dict(clocks.summary(c0, c1), whole_run=clocks.summary(0, c2))
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_sample(args.model, int8, 6, context=P)
    if rank == 0:
        print(json.dumps(line, default=lambda o: None))
    if rig.dist is not None:
        rig.dist.destroy_process_group()


def strip(d: dict) -> dict:
    return {k: v for k, v in d.items() if not k.startswith("_")}


def extra_legs(rig: Rig, args, repeats: int) -> dict:
    """Further configurations, each built, timed and released in turn.  At more than one GPU only the tensor-parallel
    configuration runs (8B fp16, batch 32, 512- and 4096-token contexts); the others are single-GPU workloads."""
    out = {}
    K, W = args.steps, args.warmup
    R = max(1, min(repeats, 3))
    xb = 32
    p8, tied8 = arch("8B")
    kb = max(16, K // 4)
    # batch 32 at a short context, then the workload's own 4096-token context (17 GB of K/V per step on one GPU)
    for name, ctx in (("decode_bs32", args.prompt), ("c4_bs32_ctx4096", 4096)):
        llm = rig.llama("8B", "float16", (ctx + (R + 1) * kb + W + 64 + 63) // 64 * 64, xb, n_layers=p8["n_layers"])
        out[name] = strip(decode_leg(rig, llm, xb, ctx, kb, W, R, tied8, False, check_steps=4))
        del llm
        rig.release()
    if rig.world > 1 or args.model != "8B" or args.quant != "float16" or LAYERS_OVERRIDE:
        return out
    # int8 weights (untied int8 output layer): batch 1, 8 and 32 at a 2048-token context, and the 2048-token prompt itself
    for b in (1, 8, 32):
        llm = rig.llama("8B", "int8", (2048 + (R + 1) * kb + W + 64 + 63) // 64 * 64, b)
        out[f"int8_bs{b}_ctx2048"] = strip(decode_leg(rig, llm, b, 2048, kb, W, R, tied8, True, check_steps=4))
        if b == 1:
            out["int8_prefill2048"] = prefill_leg(rig, llm, 1, 2048, True)
        del llm
        rig.release()
    # Llama-3.2-3B architecture: 512-token prompt, then decode; Llama-3.2-1B architecture: 32-token prompt, decode
    for size, prompt in (("3B", 512), ("1B", 32)):
        pa, tied = arch(size)
        llm = rig.llama(size, "float16", (prompt + (R + 1) * K + W + 64 + 63) // 64 * 64, 1)
        leg = strip(decode_leg(rig, llm, 1, prompt, K, W, R, tied, False, check_steps=4))
        if size == "3B":
            leg["prefill"] = prefill_leg(rig, llm, 1, prompt, False)
        out["c2_3b" if size == "3B" else "c1_1b"] = leg
        del llm
        rig.release()
    return out


def captured_traffic(model: str, quant: str, batch: int, world: int, field: str = "dram_bytes_per_launch", suffix: str = ""):
    """DRAM bytes (read + write) of one launch of the dominant kernel from the committed profiler capture of this
    workload, if there is one: profiles/traffic.json maps "<model>/<quant>/bs<batch>/tp<world>" to bytes per launch
    (and the same key + "/step" to the bytes of one decode step of the single-kernel step)."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get(f"{model}/{quant}/bs{batch}/tp{world}{suffix}", {}).get(field)
    except Exception:
        return None


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5, help="how many times the K-step timed region is repeated (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="8B", choices=["1B", "3B", "8B", "70B"])
    ap.add_argument("--quant", default="float16", choices=["float16", "int8"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0, help="reduced depth (profiling captures only; 0 = the model's own)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra legs")
    ap.add_argument("--no-parity", action="store_true", help="skip the checks against the CPU checker (profiling captures only)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    global LAYERS_OVERRIDE
    LAYERS_OVERRIDE = args.layers
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
