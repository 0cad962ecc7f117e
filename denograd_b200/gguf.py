"""GGUF checkpoints for the Llama path, on host arrays: the container (jsgrad/nn/state.ts:236-277 `gguf_load`), the
ggml block formats the reference dequantises (jsgrad/nn/state.ts:192-228 `ggml_data_to_tensor`: F32, F16, I8, I16, I32
and Q4_0, Q4_1, Q8_0, Q6_K) and the tensor-name map to the model's state dict (jsgrad/models/llama.ts:255-270
`convert_from_gguf`).  Dequantisation is float32 arithmetic with the reference's operation order; the result is what
`Llama3.load_weights` then narrows to fp16 or re-quantises to int8 / NF4 like any other checkpoint.

File layout (little endian): magic "GGUF", int32 version (2 or 3), int64 tensor count, int64 key/value count; the
key/value pairs (string key, int32 type tag, value); per tensor: name, uint32 rank, uint64 dims (innermost first), int32
ggml type, uint64 offset; then the tensor data, starting at the next multiple of `general.alignment` (32 by default).
"""
from __future__ import annotations

import struct

import numpy as np

# scalar type tags of key/value entries (jsgrad/nn/state.ts:230): tag -> struct format
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_NATIVE = {0: np.float32, 1: np.float16, 16: np.int8, 17: np.int16, 18: np.int32}
# quantised types: ggml type -> (elements per block, bytes per block)
_BLOCKS = {2: (32, 18), 3: (32, 20), 8: (32, 34), 14: (256, 210)}


def _q_to_uint8(t: np.ndarray, b: int) -> np.ndarray:
    """Unpack b-bit fields from bytes the way the reference's q_to_uint8 orders them: for input [..., n] the result is
    [..., (8/b) * n] with field j of every byte gathered before field j+1 (all low nibbles, then all high nibbles)."""
    shifts = np.arange(8 // b, dtype=np.uint8) * b
    fields = (t[..., None] >> shifts) & (0xFF >> (8 - b))  # [..., n, 8/b]
    return np.swapaxes(fields, -1, -2).reshape(*t.shape[:-1], -1)


def ggml_data_to_tensor(t: np.ndarray, n: int, ggml_type: int) -> np.ndarray:
    """`n` elements of ggml type `ggml_type` starting at byte 0 of `t` (uint8) -> a flat numpy array: the native types
    as they are, the quantised ones dequantised to float32."""
    t = np.ascontiguousarray(t, dtype=np.uint8)
    if ggml_type in _NATIVE:
        dt = np.dtype(_NATIVE[ggml_type])
        return t[:dt.itemsize * n].view(dt)
    if ggml_type not in _BLOCKS:
        raise ValueError(f"GGML type '{ggml_type}' is not supported!")
    per, nbytes = _BLOCKS[ggml_type]
    blocks = t[:(n // per) * nbytes].reshape(-1, nbytes)

    def f16(col0: int) -> np.ndarray:  # one fp16 per block, widened: [blocks, 1]
        return np.ascontiguousarray(blocks[:, col0:col0 + 2]).view(np.float16).astype(np.float32)

    if ggml_type == 2:  # Q4_0: (nibble - 8) * d
        q = _q_to_uint8(blocks[:, 2:], 4).view(np.int8) - np.int8(8)
        return (q.astype(np.float32) * f16(0)).reshape(-1)
    if ggml_type == 3:  # Q4_1: nibble * d + m
        q = _q_to_uint8(blocks[:, 4:], 4).view(np.int8)
        return (q.astype(np.float32) * f16(0) + f16(2)).reshape(-1)
    if ggml_type == 8:  # Q8_0: d * int8
        return (f16(0) * np.ascontiguousarray(blocks[:, 2:]).view(np.int8).astype(np.float32)).reshape(-1)
    # Q6_K: 128 bytes of low nibbles, 64 bytes of 2-bit high parts, 16 int8 scales, one fp16 d per 256 elements
    xl = _q_to_uint8(blocks[:, :128].reshape(-1, 2, 64), 4)
    xh = _q_to_uint8(blocks[:, 128:192].reshape(-1, 2, 32), 2) << np.uint8(4)
    q = ((xl | xh).view(np.int8) - np.int8(32)).reshape(-1, 256)
    scales = np.repeat(np.ascontiguousarray(blocks[:, 192:208]).view(np.int8), 16, axis=1)
    d = f16(208)
    return ((d * q.astype(np.float32)) * scales.astype(np.float32)).reshape(-1)


class _Reader:
    def __init__(self, data):
        self.data, self.pos = memoryview(data), 0

    def read(self, n: int) -> bytes:
        if self.pos + n > len(self.data):
            raise ValueError("GGUF file ends inside a field")
        out = bytes(self.data[self.pos:self.pos + n])
        self.pos += n
        return out

    def scalar(self, tag: int):
        fmt = _SCALARS[tag]
        return struct.unpack(fmt, self.read(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        return self.read(self.scalar(10)).decode("utf-8", errors="replace")

    def value(self, tag: int):
        if tag == 8:
            return self.string()
        if tag == 9:
            inner, n = self.scalar(5), self.scalar(10)
            return [self.value(inner) for _ in range(n)]
        if tag not in _SCALARS:
            raise ValueError(f"GGUF key/value type {tag} is unknown")
        return self.scalar(tag)


def gguf_load(data) -> tuple[dict, dict[str, np.ndarray]]:
    """(key/value metadata, {tensor name: array}) from the bytes of a GGUF file (bytes, memoryview or uint8 array).
    Shapes are the file's dims reversed, i.e. outermost first as the model expects them."""
    raw = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1)
    r = _Reader(raw)
    magic, version, n_tensors, n_kv = r.read(4), r.scalar(5), r.scalar(11), r.scalar(11)
    if magic != b"GGUF" or version not in (2, 3):
        raise ValueError(f"Invalid GGUF format, magic= {magic.decode('latin-1')}")
    kv_data: dict = {}
    for _ in range(n_kv):
        k, typ = r.string(), r.scalar(5)
        kv_data[k] = r.value(typ)
    infos = []
    for _ in range(n_tensors):
        name = r.string()
        dims = [r.scalar(10) for _ in range(r.scalar(4))]
        infos.append((name, dims, r.scalar(5), r.scalar(10)))
    align = int(kv_data.get("general.alignment") or 32)
    start = (r.pos + align - 1) // align * align
    state: dict[str, np.ndarray] = {}
    for name, dims, typ, off in infos:
        n = int(np.prod(dims, dtype=np.int64))
        state[name] = ggml_data_to_tensor(raw[start + off:], n, typ).reshape(dims[::-1])
    return kv_data, state


def convert_from_gguf(weights: dict[str, np.ndarray], n_layers: int) -> dict[str, np.ndarray]:
    """llama.cpp tensor names -> the model's state-dict names (jsgrad/models/llama.ts:255-270); the output matrix is
    the embedding table, as the reference sets it.  Names outside the map are dropped (the reference files them under
    `undefined`)."""
    keymap = {"token_embd.weight": "tok_embeddings.weight", "output_norm.weight": "norm.weight",
              "rope_freqs.weight": "rope_freqs.weight"}
    for l in range(n_layers):
        keymap[f"blk.{l}.attn_norm.weight"] = f"layers.{l}.attention_norm.weight"
        keymap[f"blk.{l}.ffn_norm.weight"] = f"layers.{l}.ffn_norm.weight"
        keymap[f"blk.{l}.attn_output.weight"] = f"layers.{l}.attention.wo.weight"
        for x in "qkv":
            keymap[f"blk.{l}.attn_{x}.weight"] = f"layers.{l}.attention.w{x}.weight"
        for x, y in (("gate", "1"), ("down", "2"), ("up", "3")):
            keymap[f"blk.{l}.ffn_{x}.weight"] = f"layers.{l}.feed_forward.w{y}.weight"
    sd = {keymap[k]: v for k, v in weights.items() if k in keymap}
    sd["output.weight"] = weights["token_embd.weight"]
    return sd
