"""Seeded synthetic weights and prompts for the benchmark workloads, generated on the device.

The workloads fix distributions, not checkpoints: fp16 weights ~N(0, 0.02), RMSNorm weights = 1, int8 weights uniform
in [-127, 127] with fp16 per-output-row scales, prompt ids uniform in [0, vocab).  Each tensor is filled by a
counter-based generator seeded from its state-dict name, so any host can regenerate the same bits (the test-suite's
CPU checker does) without moving gigabytes across PCIe.  This replaces the reference's checkpoint download
(jsgrad/models/llama3.ts:314-333), which needs a network.
"""
from __future__ import annotations

import numpy as np

from .device import Tensor
from .nn import get_state_dict

BASE_SEED = 1234
WEIGHT_STD = 0.02
INT8_SCALE_BASE = 0.02 / 73.3  # dequantised std ~ 0.02: uniform[-127,127] has std 73.3
PROMPT_SEED = 42


def name_seed(name: str, base: int = BASE_SEED) -> int:
    """64-bit FNV-1a of the tensor name, xor the base seed."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h ^ base


def _word(seed: int, c: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser of seed + (c+1)*golden — the generator's only primitive (uint64 wrap-around math)."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + (c.astype(np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def prompt_tokens(n: int, vocab: int, batch: int = 1, seed: int = PROMPT_SEED) -> np.ndarray:
    """int32 [batch, n] prompt ids uniform in [0, vocab): token i of row b is word(seed, b*n + i)."""
    c = np.arange(batch * n, dtype=np.uint64)
    hi = _word(seed, c) >> np.uint64(32)
    return ((hi * np.uint64(vocab)) >> np.uint64(32)).astype(np.int32).reshape(batch, n)


def fill_tensor(name: str, t: Tensor, base_seed: int = BASE_SEED) -> None:
    """Fill one model tensor on its device according to its name and dtype."""
    dev, seed, n = t.dev, name_seed(name, base_seed), t.numel()
    if name.endswith("norm.weight"):
        dev.call("jg_fill_const_f16", t.ptr, n, 1.0)
    elif name.endswith(".scale"):
        dev.call("jg_fill_scale_f16", t.ptr, seed, 0, n, INT8_SCALE_BASE)
    elif t.dtype == "int8":
        dev.call("jg_fill_uniform_i8", t.ptr, seed, 0, n)
    elif t.dtype == "float16":
        dev.call("jg_fill_normal_f16", t.ptr, seed, 0, n, WEIGHT_STD)
    else:
        raise TypeError(f"no synthetic fill for {name} of dtype {t.dtype}")


def fill_model(model, base_seed: int = BASE_SEED) -> dict[str, Tensor]:
    """Fill every weight of `model` (anything get_state_dict names except the RoPE table); tied tensors once.  A
    tensor-parallel model holds windows of the full tensors: each is filled with the values the full tensor has there."""
    sd = get_state_dict(model)
    shards = getattr(model, "_shards", None) or {}
    done: set[int] = set()
    for name, t in sd.items():
        if name == "freqs_cis" or t.ptr in done:
            continue
        if name in shards:
            sh = shards[name]
            seed = name_seed(sh.seed_name, base_seed)
            if name.endswith(".scale"):
                assert t.numel() == sh.rows, (name, t.shape, sh)
                t.dev.call("jg_fill_scale_f16", t.ptr, seed, sh.row0, sh.rows, INT8_SCALE_BASE)
            elif t.dtype == "int8":
                assert tuple(t.shape) == (sh.rows, sh.cols), (name, t.shape, sh)
                t.dev.call("jg_fill_uniform_i8_2d", t.ptr, seed, sh.rows, sh.cols, sh.cols_full, sh.row0, sh.col0)
            else:
                assert tuple(t.shape) == (sh.rows, sh.cols), (name, t.shape, sh)
                t.dev.call("jg_fill_normal_f16_2d", t.ptr, seed, sh.rows, sh.cols, sh.cols_full, sh.row0, sh.col0, WEIGHT_STD)
            done.add(t.ptr)
            continue
        # views of a fused allocation are filled through their own names, so each projection keeps its own stream
        fill_tensor(name, t, base_seed)
        done.add(t.ptr)
    return sd
