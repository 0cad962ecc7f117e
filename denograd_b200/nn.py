"""Layers used by the Llama path, with the reference's class names and call semantics, each backed by one kernel of
the CUDA device: Linear (jsgrad/nn/index.ts:403-412), RMSNorm (:580-589), Embedding (:600-620), Int8Linear and
Int8Embedding (jsgrad/models/llama3.ts:27-78), NF4Linear (:79-117), plus get_state_dict / load_state_dict
(jsgrad/nn/state.ts:115-179) for the tensors these classes own.
"""
from __future__ import annotations

import numpy as np

from .device import CUDA, Buffer, Device, Tensor


def _dev(device) -> CUDA:
    return device if isinstance(device, CUDA) else Device[device]


def _rows(x: Tensor) -> int:
    return x.numel() // x.shape[-1]


class Linear:
    """y = x @ W.T (no bias on this path).  ``weight`` is [out_features, in_features] fp16, uninitialised until a
    state dict is loaded (the reference draws uniform values that loading then replaces)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None, weight: Tensor | None = None):
        if bias is not False:
            raise ValueError("Linear bias is not used on the Llama path")
        self.in_features, self.out_features = in_features, out_features
        self.weight = weight if weight is not None else Tensor.empty((out_features, in_features), "float16", _dev(device))

    @property
    def scale_ptr(self) -> int:
        return 0

    def row_views(self, r0: int, r1: int) -> dict:
        """Constructor arguments of a layer of the same class over output rows [r0, r1) of this one's tensors (wq / wk /
        wv are such windows of one fused allocation)."""
        return {"weight": self.weight.view_rows(r0, r1)}

    def call(self, x: Tensor, residual: Tensor | None = None, out: Tensor | None = None) -> Tensor:
        M = _rows(x)
        y = out if out is not None else Tensor.empty(x.shape[:-1] + (self.out_features,), "float16", x.dev)
        x.dev.call("jg_linear", y.ptr, x.ptr, self.weight.ptr, self.scale_ptr, residual.ptr if residual is not None else 0,
                   M, self.out_features, self.in_features)
        return y

    __call__ = call


class Int8Linear(Linear):
    """x.dot(weight.cast(half).T * scale) — int8 weight, fp16 per-output-row scale (jsgrad/models/llama3.ts:27-35)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None, weight: Tensor | None = None,
                 scale: Tensor | None = None):
        if bias is not False:
            raise ValueError("Int8Linear bias has to be false")
        self.in_features, self.out_features = in_features, out_features
        self.weight = weight if weight is not None else Tensor.empty((out_features, in_features), "int8", _dev(device))
        self.scale = scale if scale is not None else Tensor.empty((out_features,), "float16", _dev(device))

    @property
    def scale_ptr(self) -> int:
        return self.scale.ptr

    def row_views(self, r0: int, r1: int) -> dict:
        return {"weight": self.weight.view_rows(r0, r1), "scale": self.scale.view_rows(r0, r1)}

    @staticmethod
    def quantize(tensors: dict[str, np.ndarray], quantize_embeds: bool = False) -> dict[str, np.ndarray]:
        """Int8Linear.quantize (jsgrad/models/llama3.ts:37-60) on host arrays: scale = max|row| / 127 in fp16,
        weight = round(W / scale).  The arithmetic is fp16 op by op, as in the reference graph."""
        out: dict[str, np.ndarray] = {}
        for name, v in tensors.items():
            if "feed_forward" in name or "attention.w" in name or (quantize_embeds and "tok_embeddings.weight" in name):
                assert "weight" in name
                v = v.astype(np.float16)
                scale = (np.abs(v).max(axis=1).astype(np.float16) * (np.float16(1.0) / np.float16(127.0))).astype(np.float16)
                inv = (np.float16(1.0) / scale.astype(np.float32)).astype(np.float16)
                q = np.rint((v * inv[:, None]).astype(np.float16).astype(np.float32))
                out[name] = np.clip(q, -128, 127).astype(np.int8)
                out[name.replace("weight", "scale")] = scale
            else:
                out[name] = v
        if quantize_embeds:
            out["output.weight"] = out["tok_embeddings.weight"]
            out["output.scale"] = out["tok_embeddings.scale"]
        return out


NF4_CODE = np.array([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                     -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                     0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                     0.7229568362236023, 1.0], np.float64).astype(np.float16)  # jsgrad/models/llama3.ts:80-81


def NF4Linear(block_size: int):
    """NF4Linear(block_size) -> layer class (jsgrad/models/llama3.ts:79-117): `weight` holds two 4-bit codes per byte
    (element 2i in the high nibble), `scale` one fp16 per `block_size` consecutive elements of the flattened
    [out, in] matrix; call(x) = x.linear(half(CODE[code] * scale).reshape(out, in).T).  On this device the packed form
    is what stays resident; a call dequantises the matrix into a scratch shared by all NF4 layers of the device
    (jg_dequant_nf4_f16) and runs the fp16 projection on it."""
    scratch: dict[str, Tensor] = {}

    class _NF4Linear:
        nf4_block = block_size

        def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None,
                     weight: Tensor | None = None, scale: Tensor | None = None):
            if bias:
                raise ValueError("bias not supported")
            if (in_features * out_features) % 32 or in_features % block_size or block_size % 2:
                raise ValueError(f"NF4Linear: {out_features} x {in_features} does not divide into blocks of {block_size}")
            self.in_features, self.out_features = in_features, out_features
            n = out_features * in_features
            self.weight = weight if weight is not None else Tensor.empty((n // 2,), "uint8", _dev(device))
            self.scale = scale if scale is not None else Tensor.empty((n // block_size, 1), "float16", _dev(device))

        @property
        def scale_ptr(self) -> int:
            return 0  # the projection kernels see the dequantised fp16 copy

        def row_views(self, r0: int, r1: int) -> dict:
            k = self.in_features
            return {"weight": self.weight.view_rows(r0 * k // 2, r1 * k // 2),
                    "scale": self.scale.view_rows(r0 * k // block_size, r1 * k // block_size)}

        def dequantised(self) -> Tensor:
            """fp16 [out, in] in the shared scratch (valid until the next NF4 layer of this device is called)."""
            dev, n = self.weight.dev, self.out_features * self.in_features
            t = scratch.get(dev.device)
            if t is None or t.numel() < n:
                t = scratch[dev.device] = Tensor.empty((n,), "float16", dev)
            dev.call("jg_dequant_nf4_f16", t.ptr, self.weight.ptr, self.scale.ptr, n, block_size)
            return t

        def call(self, x: Tensor, residual: Tensor | None = None, out: Tensor | None = None) -> Tensor:
            M = _rows(x)
            y = out if out is not None else Tensor.empty(x.shape[:-1] + (self.out_features,), "float16", x.dev)
            w = self.dequantised()
            x.dev.call("jg_linear", y.ptr, x.ptr, w.ptr, 0, residual.ptr if residual is not None else 0,
                       M, self.out_features, self.in_features)
            return y

        __call__ = call

        @staticmethod
        def quantize(state_dict: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
            """NF4Linear.quantize (jsgrad/models/llama3.ts:96-113) on host arrays, fp16 op by op: per block
            scale = max|v|, code = argmin_c |half(half(v * half(1 / scale)) - CODE[c])| (lowest index among equals)."""
            out: dict[str, np.ndarray] = {}
            for k, v in state_dict.items():
                if "feed_forward" in k or "attention.w" in k:
                    g = np.asarray(v, dtype=np.float16).reshape(-1, block_size)
                    scale = np.abs(g).max(axis=1, keepdims=True).astype(np.float16)
                    with np.errstate(divide="ignore", invalid="ignore"):
                        inv = (np.float32(1.0) / scale.astype(np.float32)).astype(np.float16)
                        q = (g.astype(np.float32) * inv.astype(np.float32)).astype(np.float16)
                        dist = np.abs((q[..., None].astype(np.float32) - NF4_CODE.astype(np.float32)).astype(np.float16))
                    coded = dist.argmin(axis=-1).astype(np.uint8).reshape(-1)
                    out[k] = (coded[0::2] * np.uint8(16) + coded[1::2]).astype(np.uint8)
                    out[k.replace(".weight", ".scale")] = scale
                else:
                    out[k] = v
            return out

    return _NF4Linear


class RMSNorm:
    def __init__(self, dim: int, eps: float = 1e-6, device=None):
        self.eps = eps
        self.weight = Tensor(np.ones((dim,), np.float16), device=_dev(device))

    def call(self, x: Tensor, out: Tensor | None = None) -> Tensor:
        y = out if out is not None else Tensor.empty(x.shape, "float16", x.dev)
        x.dev.call("jg_rmsnorm", y.ptr, x.ptr, self.weight.ptr, _rows(x), x.shape[-1], self.eps)
        return y

    __call__ = call


class Embedding:
    def __init__(self, vocab_size: int, embed_size: int, device=None, weight: Tensor | None = None):
        self.vocab_size, self.embed_size = vocab_size, embed_size
        self.weight = weight if weight is not None else Tensor.empty((vocab_size, embed_size), "float16", _dev(device))

    @property
    def scale_ptr(self) -> int:
        return 0

    def call(self, idx: Tensor, out: Tensor | None = None) -> Tensor:
        assert idx.dtype == "int32"
        y = out if out is not None else Tensor.empty(tuple(idx.shape) + (self.embed_size,), "float16", idx.dev)
        idx.dev.call("jg_embed", y.ptr, idx.ptr, self.weight.ptr, self.scale_ptr, idx.numel(), self.embed_size, self.vocab_size)
        return y

    __call__ = call


class Int8Embedding(Embedding):
    def __init__(self, vocab_size: int, embed_size: int, device=None):
        self.vocab_size, self.embed_size = vocab_size, embed_size
        self.weight = Tensor.empty((vocab_size, embed_size), "int8", _dev(device))
        self.scale = Tensor.empty((vocab_size,), "float16", _dev(device))

    @property
    def scale_ptr(self) -> int:
        return self.scale.ptr


# ---------------------------------------------------------------------------------------------- state dicts
def get_state_dict(obj, prefix: str = "") -> dict[str, Tensor]:
    """Walk attributes / lists and collect Tensors under dotted names (jsgrad/nn/state.ts:115-140)."""
    if isinstance(obj, Tensor):
        return {prefix.rstrip("."): obj}
    out: dict[str, Tensor] = {}
    if isinstance(obj, (list, tuple)):
        for i, x in enumerate(obj):
            out.update(get_state_dict(x, f"{prefix}{i}."))
    elif isinstance(obj, dict):
        for k, x in obj.items():
            out.update(get_state_dict(x, f"{prefix}{k}."))
    elif hasattr(obj, "__dict__") and not isinstance(obj, (CUDA, Buffer)):
        for k, x in vars(obj).items():
            if k.startswith("_"):
                continue
            out.update(get_state_dict(x, f"{prefix}{k}."))
    return out


def load_state_dict(model, state_dict: dict[str, np.ndarray], strict: bool = True) -> None:
    """Copy host arrays into the model's tensors by name (jsgrad/nn/state.ts:159-179): shapes must match; with
    ``strict`` every model tensor must be present."""
    model_state = get_state_dict(model)
    for k, v in model_state.items():
        if k not in state_dict:
            if strict:
                raise KeyError(f"{k} is missing from the state dict")
            continue
        src = state_dict[k]
        if tuple(src.shape) != tuple(v.shape):
            raise ValueError(f"Shape mismatch in layer {k}: Expected shape {v.shape}, but found {tuple(src.shape)} in state dict.")
        v.assign(src)
