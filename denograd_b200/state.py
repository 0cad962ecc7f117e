"""Checkpoint files for the Llama path: the safetensors container and the Hugging Face -> Llama name / layout
conversion, on host arrays (GGUF files: gguf.py).  Counterpart of jsgrad/nn/state.ts:22-96 (safe_load / safe_save) and
jsgrad/models/llama.ts:224-253,272-279 (convert_from_huggingface, fix_bf16); `Llama3.load_weights` in llama3.py strings
them together the way Llama3.load does (jsgrad/models/llama3.ts:201-258), minus the download.

A safetensors file is: 8 bytes little-endian header length n, n bytes of JSON {name: {dtype, shape, data_offsets}},
then the tensors' bytes back to back (offsets are relative to the end of the header).
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

# safetensors dtype tag -> numpy dtype (jsgrad/nn/state.ts:22-36); BF16 has no numpy type and is widened on load
_SAFE_DTYPES = {"BOOL": np.bool_, "I8": np.int8, "U8": np.uint8, "I16": np.int16, "U16": np.uint16, "I32": np.int32,
                "U32": np.uint32, "I64": np.int64, "U64": np.uint64, "F16": np.float16, "F32": np.float32, "F64": np.float64}
_SAFE_TAGS = {np.dtype(v): k for k, v in _SAFE_DTYPES.items()}


def bf16_to_f16(raw: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) -> float16 through float32, the reference's fix_bf16 (cast to float32, then to
    float16; jsgrad/models/llama.ts:272-276): the widening is exact, the narrowing rounds to nearest even."""
    with np.errstate(over="ignore"):  # bf16 magnitudes beyond the fp16 range become infinities, as a cast does
        return (raw.astype(np.uint32) << 16).view(np.float32).astype(np.float16)


def safe_load(path: str) -> dict[str, np.ndarray]:
    """Read every tensor of a .safetensors file (memory-mapped; BF16 tensors come back as float16)."""
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n <= 0 or 8 + n > size:
            raise ValueError(f"{path}: header length {n} exceeds the file ({size} bytes)")
        meta = json.loads(f.read(n).decode("utf-8"))
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + n)
    out: dict[str, np.ndarray] = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        if not (0 <= lo <= hi <= data.size):
            raise ValueError(f"{path}: tensor {name} lies outside the file")
        raw, shape, tag = data[lo:hi], tuple(info["shape"]), info["dtype"]
        if tag == "BF16":
            arr = bf16_to_f16(raw.view(np.uint16))
        elif tag in _SAFE_DTYPES:
            arr = raw.view(_SAFE_DTYPES[tag])
        else:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {tag}")
        if int(np.prod(shape, dtype=np.int64)) != arr.size:
            raise ValueError(f"{path}: tensor {name} has {arr.size} elements, its shape {shape} says otherwise")
        out[name] = arr.reshape(shape)
    return out


def safe_save(tensors: dict[str, np.ndarray], path: str, metadata: dict | None = None) -> None:
    """Write host arrays as a .safetensors file (header padded with spaces to a multiple of 8 bytes)."""
    header: dict = {"__metadata__": metadata} if metadata else {}
    offset = 0
    arrays = {k: np.ascontiguousarray(v) for k, v in tensors.items()}
    for k, v in arrays.items():
        if v.dtype not in _SAFE_TAGS:
            raise TypeError(f"{k}: dtype {v.dtype} has no safetensors tag")
        header[k] = {"dtype": _SAFE_TAGS[v.dtype], "shape": list(v.shape), "data_offsets": [offset, offset + v.nbytes]}
        offset += v.nbytes
    j = json.dumps(header, separators=(",", ":")).encode("utf-8")
    j += b" " * (-len(j) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(j)))
        f.write(j)
        for v in arrays.values():
            f.write(v.tobytes())


def load_checkpoint(path: str) -> dict[str, np.ndarray]:
    """One .safetensors file, or a sharded checkpoint through its *.index.json (weight_map: tensor name -> file name,
    files next to the index), as Llama3._load resolves them (jsgrad/models/llama3.ts:201-213)."""
    if path.endswith(".index.json"):
        with open(path) as f:
            weight_map = json.load(f)["weight_map"]
        base = os.path.dirname(path)
        parts = {fn: safe_load(os.path.join(base, fn)) for fn in sorted(set(weight_map.values()))}
        return {k: parts[fn][k] for k, fn in weight_map.items()}
    if path.endswith(".safetensors"):
        return safe_load(path)
    if path.endswith(".gguf"):
        from .gguf import gguf_load
        return gguf_load(np.memmap(path, dtype=np.uint8, mode="r"))[1]
    raise ValueError(f"{path}: expected a .safetensors file, a *.index.json of safetensors shards, or a .gguf file")


def _permute(v: np.ndarray, n_heads: int) -> np.ndarray:
    """Rows of a Hugging Face q/k projection hold each head's rotary pairs as two halves (first all even members, then
    all odd ones); the Llama layout interleaves them.  [H, 2, hd/2, in] -> [H, hd/2, 2, in]
    (jsgrad/models/llama.ts:225-227)."""
    out_f, in_f = v.shape
    return v.reshape(n_heads, 2, out_f // n_heads // 2, in_f).transpose(0, 2, 1, 3).reshape(out_f, in_f)


def convert_from_huggingface(weights: dict[str, np.ndarray], n_layers: int, n_heads: int, n_kv_heads: int,
                             permute_layers: bool = True) -> dict[str, np.ndarray]:
    """Hugging Face tensor names -> the model's state-dict names, q/k rows permuted to the interleaved rotary layout
    (jsgrad/models/llama.ts:224-253).  Unknown names raise (the reference would store them under `undefined`)."""
    keymap = {"model.embed_tokens.weight": "tok_embeddings.weight", "model.norm.weight": "norm.weight",
              "lm_head.weight": "output.weight"}
    for l in range(n_layers):
        keymap[f"model.layers.{l}.input_layernorm.weight"] = f"layers.{l}.attention_norm.weight"
        keymap[f"model.layers.{l}.post_attention_layernorm.weight"] = f"layers.{l}.ffn_norm.weight"
        for x in "qkvo":
            keymap[f"model.layers.{l}.self_attn.{x}_proj.weight"] = f"layers.{l}.attention.w{x}.weight"
        for x, y in (("gate", "1"), ("down", "2"), ("up", "3")):
            keymap[f"model.layers.{l}.mlp.{x}_proj.weight"] = f"layers.{l}.feed_forward.w{y}.weight"
    sd: dict[str, np.ndarray] = {}
    for k, v in weights.items():
        if ".rotary_emb." in k:
            continue
        if k not in keymap:
            raise KeyError(f"{k}: not a tensor of a Llama checkpoint in Hugging Face naming")
        if permute_layers and "model.layers" in k:
            if "q_proj" in k:
                v = _permute(v, n_heads)
            elif "k_proj" in k:
                v = _permute(v, n_kv_heads)
        sd[keymap[k]] = v
    return sd
