"""The inputs of the reference's own hot-path test, regenerated from its source.

test/models/llama.test.ts:24-99 of the reference builds `Transformer(2048, 8192, 32, 16, 1e-5, 128256, ..., n_kv_heads 8,
rope_theta 500000, max_context 8192, jit false)` after `Tensor.manual_seed(4)` and calls `forward([[459]], start_pos 7,
temperature 0.85, top_k 0, top_p 0, alpha 0, 0)` (and `[[271]]` at start_pos 4).  The expected output lives in an
un-vendored Python dependency, so nothing here is a golden vector; what *can* be reproduced are the weights and the
uniform sample, because they come from the threefry stream of Tensor.rand (jsgrad/tensor.ts:796-843) in constructor
order (jsgrad/models/llama.ts:46-57,103-107,114-122,193-199):

  per layer: wq, wk, wv, wo, w1, w2, w3  — nn.Linear: uniform(-1/sqrt(in), 1/sqrt(in)) = rand * (2b) + (-b), float32
  then tok_embeddings — glorot_uniform: (rand * 2 + (-1)) * sqrt(6 / (vocab + dim)); then output — nn.Linear
  norms are ones.  The draw inside `sample` is the next Tensor.rand([1, 1, 1]).

The reference runs this test in float32; this device and its checker compute in fp16, so the float32 weights are
narrowed once (round to nearest even).  TEST INFRASTRUCTURE: uses the checker's threefry (oracle/sample_oracle.c).
"""
from __future__ import annotations

import hashlib

import numpy as np

from oracle import oracle as O

ARCH = {"dim": 2048, "hidden_dim": 8192, "n_heads": 32, "n_layers": 16, "norm_eps": 1e-5, "vocab_size": 128256,
        "n_kv_heads": 8, "rope_theta": 500000}
CALLS = [(459, 7), (271, 4)]  # (token, start_pos) of the test's two cases
TEMPERATURE = 0.85


class RandStream:
    """Tensor.rand call by call for one device after manual_seed(seed) (first device name seen: hash of 0)."""

    def __init__(self, seed: int):
        self.seed0 = int.from_bytes(hashlib.sha256((0).to_bytes(4, "big")).digest(), "big") % (1 << 32)
        self.seed1, self.counter, self.first = seed & 0xFFFFFFFF, 0, True

    def rand(self, numel: int) -> np.ndarray:
        if self.first:
            self.first = False
        else:
            self.counter = (self.counter + numel) & 0xFFFFFFFF
        return O.threefry_rand(self.seed0, self.seed1, self.counter, numel)


def _uniform(r: RandStream, shape, low: float, high: float) -> np.ndarray:
    u = r.rand(int(np.prod(shape)))
    w = u * np.float32(high - low)          # rand.mul(high - low, reverse)
    w += np.float32(low)                    # .add(low)
    return w.reshape(shape)


def state_dict(seed: int = 4, n_layers: int | None = None):
    """(name -> fp16 array in the model's state-dict names, the uniform sample `sample` will draw)."""
    p = ARCH
    d, f, V, hd = p["dim"], p["hidden_dim"], p["vocab_size"], p["dim"] // p["n_heads"]
    kv = p["n_kv_heads"] * hd
    r = RandStream(seed)
    sd: dict[str, np.ndarray] = {}
    L = p["n_layers"]
    for l in range(L):
        for name, (o, i) in (("attention.wq", (d, d)), ("attention.wk", (kv, d)), ("attention.wv", (kv, d)), ("attention.wo", (d, d)),
                             ("feed_forward.w1", (f, d)), ("feed_forward.w2", (d, f)), ("feed_forward.w3", (f, d))):
            b = 1.0 / np.sqrt(i)
            w = _uniform(r, (o, i), -b, b)
            if n_layers is None or l < n_layers:
                sd[f"layers.{l}.{name}.weight"] = w.astype(np.float16)
        if n_layers is None or l < n_layers:
            sd[f"layers.{l}.attention_norm.weight"] = np.ones(d, np.float16)
            sd[f"layers.{l}.ffn_norm.weight"] = np.ones(d, np.float16)
    emb = _uniform(r, (V, d), -1.0, 1.0) * np.float32((6.0 / (V + d)) ** 0.5)
    sd["tok_embeddings.weight"] = emb.astype(np.float16)
    b = 1.0 / np.sqrt(d)
    sd["output.weight"] = _uniform(r, (V, d), -b, b).astype(np.float16)
    sd["norm.weight"] = np.ones(d, np.float16)
    u = float(r.rand(1)[0])  # multinomial's Tensor.rand([1, 1, 1])
    return sd, u
