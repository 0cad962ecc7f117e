"""Benchmark of the Llama-3 greedy-decode hot path on the CUDA device (and of the CPU reference arm).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                  [--model 8B] [--quant float16|int8] [--batch B] [--prompt P]

A step is one decode step (one new token per batch row) of the whole model.  Default workload: Llama-3.1-8B
architecture, fp16 weights ~N(0, 0.02) (seeded, generated on the device), batch 1, 512-token seeded prompt already
in the KV cache, greedy decoding.  One JSON line is printed by rank 0:

  value      decode tokens/s with everything resident in HBM: the captured step replays back to back and feeds its own
             token back on the device (timed with CUDA events on the launching stream);
  e2e        the same metric through the public per-token API: token ids and positions are copied up from page-locked
             host memory, the step runs, the chosen ids are read back — every step, as the reference's chat loop does;
  roofline   the dominant kernel (the weight-streaming matrix-vector kernel, timed alone on the gate/up projection
             of every layer in turn) against the measured HBM copy bandwidth; `step` carries the same figure for the
             whole decode step (all weights + KV read once per step);
  cpu_baseline  the CPU restatement of the reference's CLANG path (oracle/), timed on this host's cores on a bounded
             sample: full-width 1- and 4-layer slices of the same architecture, extrapolated linearly in depth.

`--impl reference` times that CPU restatement as the reference arm (the reference itself needs a JS runtime and
clang, neither of which exists here).
"""
from __future__ import annotations

import argparse
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


def measured_peaks() -> tuple[float, str]:
    """HBM GB/s denominator: the driver-measured copy bandwidth if present, else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
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

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()  # the exact child we started
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
            self.t.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ workload sizes
LAYERS_OVERRIDE = 0


def arch(model: str):
    from denograd_b200.llama3 import MODEL_PARAMS
    p = dict(MODEL_PARAMS[model]["args"])
    if LAYERS_OVERRIDE:
        p["n_layers"] = LAYERS_OVERRIDE
    return p, MODEL_PARAMS[model]["tied"]


def weight_bytes(p: dict, tied: bool, int8: bool) -> int:
    """Bytes of weights one decode step streams: every projection once, the output matrix once (the embedding
    gather touches one row per token)."""
    d, hd = p["dim"], p["dim"] // p["n_heads"]
    kv, f, V, L = p["n_kv_heads"] * hd, p["hidden_dim"], p["vocab_size"], p["n_layers"]
    params = L * (2 * d * d + 2 * kv * d + 3 * f * d) + V * d
    rows = L * (2 * d + 2 * kv + 2 * f + d) + V  # scale entries (one fp16 per output row) for int8
    return params * (1 if int8 else 2) + (rows * 2 if int8 else 0) + L * 2 * d * 2 + d * 2  # + norm weights


def kv_bytes_per_token(p: dict) -> int:
    hd = p["dim"] // p["n_heads"]
    return 2 * p["n_layers"] * p["n_kv_heads"] * hd * 2


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(model: str, int8: bool, steps: int, warmup: int) -> dict:
    """Times the CPU restatement (oracle/) on full-width 1- and 4-layer slices of `model`, batch 1, and extrapolates
    the per-token time of the full depth: t(L) = t_head + L * t_layer."""
    from oracle import oracle as O  # the checker, used here only as the timed CPU baseline
    from tests.util import build_oracle
    from denograd_b200 import synth
    p, tied = arch(model)
    steps = max(6, min(steps, 48))
    warmup = max(1, min(warmup, 4))
    times = {}
    for L in (1, 4):
        q = dict(p); q["n_layers"] = L
        m = build_oracle(q, max_context=warmup + steps + 8, max_batch=1, int8=int8, tied=tied)
        toks = synth.prompt_tokens(warmup + steps, p["vocab_size"])
        for i in range(warmup):
            m.forward(toks[:, i:i + 1], i)
        t0 = time.perf_counter()
        for i in range(warmup, warmup + steps):
            m.forward(toks[:, i:i + 1], i)
        times[L] = (time.perf_counter() - t0) / steps
        m.close()
    t_layer = max((times[4] - times[1]) / 3.0, 1e-9)
    t_head = max(times[1] - t_layer, 0.0)
    t_full = t_head + p["n_layers"] * t_layer
    cores = int(os.environ.get("OMP_NUM_THREADS") or os.cpu_count() or 1)
    return {"value": 1.0 / t_full, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": (f"{model} architecture, batch 1: {steps} greedy steps each on full-width 1-layer and 4-layer slices "
                       f"(embedding + layers + final norm + {p['vocab_size']}-row output), short context; "
                       f"per-token time extrapolated to {p['n_layers']} layers as t_head + L*t_layer "
                       f"(t_head {t_head * 1e3:.1f} ms, t_layer {t_layer * 1e3:.1f} ms); OpenMP over output rows on all "
                       f"host cores (the reference's generated C itself is single-threaded)"),
            "ms_per_token_est": t_full * 1e3}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    int8 = args.quant == "int8"
    cb = cpu_sample(args.model, int8, args.steps, args.warmup)
    p, tied = arch(args.model)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_token_est"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 weights, f32 accumulate", "data": "synthetic",
            "config": workload_config(args, p), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(args, p) -> dict:
    return {"workload": (f"Llama-3.1-{args.model} architecture greedy decode, {args.quant} weights, batch {args.batch}, "
                         f"{args.prompt}-token seeded prompt in the KV cache"),
            "batch": args.batch, "prompt_tokens": args.prompt, "weights": args.quant, "layers": p["n_layers"],
            "l2": "inputs larger than L2: every step streams all weights (GBs) once, no flush needed",
            "parallelism": f"tp{args.gpus}" + ("" if args.gpus == 1 else
                            ": heads / FFN width / vocabulary sharded; fp32 all-reduce after wo and w2 over NVLink peer memory inside "
                            "the projection kernel (NCCL for messages above 128 KB)")}


# ------------------------------------------------------------------------------------------------ GPU arm
def run_gpu(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from denograd_b200 import synth
    from denograd_b200.device import Device, Tensor
    from denograd_b200.llama3 import Llama3

    int8 = args.quant == "int8"
    p, tied = arch(args.model)
    B, P, K, W = args.batch, args.prompt, args.steps, args.warmup
    max_ctx = P + 2 * (K + W) + 16
    max_ctx = (max_ctx + 63) // 64 * 64
    dev_name = "CUDA" if local_rank == 0 else f"CUDA:{local_rank}"
    tp = None
    if world > 1:
        # tensor parallel over the ranks: rank 0 makes the NCCL id, torch.distributed carries it to the others
        from denograd_b200.multi import TensorParallel
        box = [TensorParallel.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        tp = TensorParallel(Device[dev_name], rank, world, box[0])
        if os.environ.get("JG_TP_PEER", "1") != "0":
            from denograd_b200.multi import exchange_via_torch
            tp.open_peers(exchange_via_torch)  # small all-reduces as one kernel over NVLink peer memory
    xb = 0 if args.no_extra else 32  # batch of the extra batched-decode leg
    llm = Llama3(size=args.model, quantize=args.quant, max_context=max_ctx, max_batch=max(B, xb), device=dev_name,
                 n_layers=p["n_layers"], tp=tp).load_synthetic()
    dev = llm.model.dev
    model = llm.model

    def barrier():
        dev.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- untimed set-up: the prompt goes through the model in one multi-position forward (fills the KV cache)
    prompt = synth.prompt_tokens(P, p["vocab_size"], batch=B, seed=synth.PROMPT_SEED)
    first = llm.prefill(prompt).numpy()
    pos0 = llm.start_pos

    # ---- value: device-resident loop (graph replay, token fed back on the device)
    model.decode_loop(first, pos0, W, collect=False)  # warm-up steps (also captures the step)
    barrier()
    launches0 = dev.launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        dev.timer_start()
        model.decode_loop(first, pos0 + W, K, collect=False, resume=True)
        secs = dev.timer_stop()
        barrier()
    launches = dev.launch_count() - launches0
    secs = max_over_ranks(secs)
    value = B * K / secs  # one model sharded over the ranks: the job's tokens are the batch's tokens

    # ---- e2e: public per-token API with host buffers (pinned H2D of ids + positions, D2H of the chosen ids)
    llm.start_pos = pos0 + W + K
    tok = model._workspace(B).next_tokens.numpy()
    for _ in range(W):
        tok = model.call_host(tok.reshape(B, 1), llm.start_pos); llm.start_pos += 1
    barrier()
    dev.timer_start()
    for _ in range(K):
        tok = model.call_host(tok.reshape(B, 1), llm.start_pos); llm.start_pos += 1
    e2e_secs = max_over_ranks(dev.timer_stop())
    barrier()
    e2e_value = B * K / e2e_secs

    # ---- roofline of the dominant kernel, timed alone: gate/up projection (norm + two matrices + SwiGLU) of every
    #      layer in turn, so that consecutive launches never find their weights in L2
    peak, peak_kind = measured_peaks()
    ws = model._workspace(B)
    d, f = p["dim"], p["hidden_dim"] // world  # f: this rank's share of the FFN width

    from denograd_b200.llama import _norm_first
    big = _norm_first(B, int8)  # the projection takes pre-normalised rows and runs on the tensor cores

    def gateup(layer):
        ff = layer.feed_forward
        # above 8 rows the projection takes pre-normalised rows (ws.xn) and runs on the tensor cores
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

    # DRAM bytes of one gate/up launch from the committed ncu capture (profiles/gemv_kernel_8b_fp16_bs1.md): read +
    # write of the 8B fp16 batch-1 shape; other shapes have no capture yet
    traffic = 239192832 if (args.model == "8B" and not int8 and B == 1 and world == 1) else None
    t_mid = pos0 + W + K / 2.0  # mean cached length over the timed steps
    step_bytes = (weight_bytes(p, tied, int8) + B * t_mid * kv_bytes_per_token(p)) / world + B * d * 2  # per GPU
    step_gbs = step_bytes / (secs / K) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": secs / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 activations, f32 accumulate, " + ("i8 weights" if int8 else "f16 weights"), "data": "synthetic",
        "config": workload_config(args, p),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 4 * B,
                "ms_per_step": e2e_secs / K * 1e3},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": (("gemm_small_kernel (mma.sync, gate/up + SwiGLU instantiation)" if (int8 or B < 9) else "gemm_tc_kernel (tcgen05, gate/up + SwiGLU instantiation)") if big else "gemv_kernel (norm + gate/up + SwiGLU instantiation)"), "achieved": k_gbs,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": k_gbs / peak, "traffic": traffic,
                     "bytes_per_launch": k_bytes, "us_per_launch": k_secs * 1e6,
                     "step": {"bytes_per_step": step_bytes, "achieved": step_gbs, "frac": step_gbs / peak,
                              "hbm_roofline_tok_s": B * peak * 1e9 / step_bytes, "per_gpu": True}},
    }
    # ---- extra legs of the same metric family: prompt processing (one multi-position forward) and batch-32 decode
    if not args.no_extra:
        extra = {}
        flops_per_tok = 2 * (weight_bytes(p, tied, int8) // (1 if int8 else 2)) / world  # 2 flops per weight, per GPU
        tf_peak = 1636.2
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
                tf_peak = float(json.load(fh)["bf16_tflops"])
        except Exception:
            pass
        pl = prompt[:1, :P]
        llm.reset(); llm.prefill(pl); dev.synchronize()  # warm-up (kernels' attributes, workspaces)
        reps = 3
        barrier()
        dev.timer_start()
        for _ in range(reps):
            llm.reset()
            llm.prefill(pl)
        pf = max_over_ranks(dev.timer_stop()) / reps
        extra["prefill"] = {"tok_s": P / pf, "ms": pf * 1e3, "prompt_tokens": P, "batch": 1,
                            "tflops_per_gpu": flops_per_tok * P / pf / 1e12, "frac_of_measured_bf16_peak": flops_per_tok * P / pf / 1e12 / tf_peak,
                            "how": ("Transformer.forward over the whole prompt in chunks of up to 2048 rows: each int8 matrix dequantised once per chunk into an fp16 copy, tcgen05/TMA projections on the copy, tensor-core causal attention" if int8 else
                                    "Transformer.forward over the whole prompt in chunks of up to 2048 rows: tcgen05/TMA projections, tensor-core causal attention")}
        if xb:
            pb = synth.prompt_tokens(P, p["vocab_size"], batch=xb, seed=synth.PROMPT_SEED)
            llm.reset()
            first_b = llm.prefill(pb).numpy()
            model.decode_loop(first_b, llm.start_pos, W, collect=False)
            barrier()
            kb = max(8, K // 4)
            dev.timer_start()
            model.decode_loop(first_b, llm.start_pos + W, kb, collect=False, resume=True)
            sb = max_over_ranks(dev.timer_stop())
            tb = llm.start_pos + W + kb / 2.0
            bytes_b = (weight_bytes(p, tied, int8) + xb * tb * kv_bytes_per_token(p)) / world + xb * d * 2
            extra["decode_bs32"] = {"tok_s": xb * kb / sb, "ms_per_step": sb / kb * 1e3, "batch": xb, "steps": kb,
                                    "context": int(tb), "frac_of_hbm_roofline": bytes_b / (sb / kb) / 1e9 / peak}
        line["extra"] = extra
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_sample(args.model, int8, 8, 2)
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="8B", choices=["1B", "3B", "8B", "70B"])
    ap.add_argument("--quant", default="float16", choices=["float16", "int8"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0, help="reduced depth (profiling captures only; 0 = the model's own)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the prefill and batch-32 legs")
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
