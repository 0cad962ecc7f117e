"""Llama3 driver on the CUDA device — Python mirror of jsgrad/models/llama3.ts (MODEL_PARAMS :119-132, the Llama3
class :170-338): construction per size / quantisation with the reference's defaults, weight loading into the device,
prefill with prefix reuse, the chat loop with stop tokens and usage accounting, and greedy generation for the seeded
workloads.  Checkpoint download is not part of this path (no network); the tokenizer's vocabulary file is passed in.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np

from . import synth
from .device import Device, Tensor
from .llama import Transformer
from .nn import Embedding, Int8Embedding, Int8Linear, Linear, NF4Linear, load_state_dict

MODEL_PARAMS = {
    "1B": {"args": {"dim": 2048, "n_heads": 32, "n_kv_heads": 8, "n_layers": 16, "norm_eps": 1e-5, "rope_theta": 500000,
                    "vocab_size": 128256, "hidden_dim": 8192}, "files": 1, "tied": True},
    # not in the reference's table; Llama-3.2-3B architecture as the 3B workload states it
    "3B": {"args": {"dim": 3072, "n_heads": 24, "n_kv_heads": 8, "n_layers": 28, "norm_eps": 1e-5, "rope_theta": 500000,
                    "vocab_size": 128256, "hidden_dim": 8192}, "files": 1, "tied": True},
    "8B": {"args": {"dim": 4096, "n_heads": 32, "n_kv_heads": 8, "n_layers": 32, "norm_eps": 1e-5, "rope_theta": 500000,
                    "vocab_size": 128256, "hidden_dim": 14336}, "files": 1, "tied": False},
    "70B": {"args": {"dim": 8192, "n_heads": 64, "n_kv_heads": 8, "n_layers": 80, "norm_eps": 1e-5, "rope_theta": 500000,
                     "vocab_size": 128256, "hidden_dim": 28672}, "files": 8, "tied": False},
}


@dataclass
class Llama3Usage:
    """jsgrad/models/llama3.ts:159-164."""
    input_tokens: int = 0
    output_tokens: int = 0
    time_to_first_token: float = 0.0
    tokens_per_second: float = 0.0


@dataclass
class Llama3:
    """``Llama3(size=..., quantize=...)`` builds the Transformer with the reference's class injection
    (Int8Linear / Int8Embedding for 'int8', NF4Linear(64) for 'nf4': jsgrad/models/llama3.ts:190-200) and its defaults:
    temperature 0.95, top_k 0, top_p 0, alpha_f 0, alpha_p 0, max_context 8192.  Greedy decoding, which the benchmark
    workloads prescribe, is ``temperature=0``."""
    size: str = "1B"
    quantize: str | None = "float16"  # 'float16' | 'int8' | 'nf4'
    max_context: int = 8192
    device: str | None = None
    temperature: float = 0.95
    top_k: int = 0
    top_p: float = 0.0
    alpha_f: float = 0.0
    alpha_p: float = 0.0
    max_batch: int = 1
    page_size: int = 64
    fused: bool = True
    jit: bool = True
    n_layers: int | None = None  # override the depth (reduced-depth slices of a big architecture for checks)
    tied_output: bool | None = None
    tp: object | None = None  # denograd_b200.multi.TensorParallel: this process is one rank of a sharded model
    args: dict = field(default_factory=dict)
    last_seen_toks: list = field(default_factory=list)
    tokenizer: object | None = None  # denograd_b200.tokenizer.Tokenizer, needed by _system / chat only

    def __post_init__(self):
        if self.quantize not in ("float16", "int8", "nf4", None):
            raise ValueError(f"quantize={self.quantize!r}: expected 'float16', 'int8' or 'nf4'")
        if self.quantize == "nf4":
            if self.tp is not None:
                raise NotImplementedError("NF4 weights under tensor parallelism")
            self.fused = False  # NF4 layers dequantise per call: the per-op block path
        p = dict(MODEL_PARAMS[self.size]["args"])
        p.update(self.args)
        if self.n_layers is not None:
            p["n_layers"] = self.n_layers
        self.params = p
        int8 = self.quantize == "int8"
        self.linear = Int8Linear if int8 else (NF4Linear(64) if self.quantize == "nf4" else Linear)
        self.embedding = Int8Embedding if int8 else Embedding
        self.quantize_embeds = int8
        tied = MODEL_PARAMS[self.size]["tied"] if self.tied_output is None else self.tied_output
        self.model = Transformer(p["dim"], p["hidden_dim"], p["n_heads"], p["n_layers"], p["norm_eps"], p["vocab_size"],
                                 self.linear, self.embedding, p["n_kv_heads"], p["rope_theta"], self.max_context, self.jit,
                                 device=Device[self.device], max_batch=self.max_batch, page_size=self.page_size,
                                 tied_output=tied, fused=self.fused, tp=self.tp)
        self.usage = Llama3Usage()
        self.start_pos = 0

    # ---- weights
    def load_state_dict(self, weights: dict[str, np.ndarray]) -> "Llama3":
        """Host arrays -> device tensors by name, non-strict like the reference (jsgrad/models/llama3.ts:258-260)."""
        load_state_dict(self.model, weights, strict=False)
        return self

    def load_weights(self, path: str) -> "Llama3":
        """Weights from a checkpoint on disk, the tail of Llama3.load (jsgrad/models/llama3.ts:220-260) without the
        download: read the .safetensors file (or the shards named by its .index.json) or the .gguf file (ggml
        blocks dequantised on the host), map Hugging Face / llama.cpp names and the Hugging Face q/k row layout to the model's, narrow bf16 to fp16, cast to fp16 or quantise to int8 with the reference's
        arithmetic, cut this rank's windows under tensor parallelism, and copy by name (non-strict)."""
        from .state import convert_from_huggingface, load_checkpoint
        p = self.params
        w = load_checkpoint(path)
        if "model.embed_tokens.weight" in w:
            w = convert_from_huggingface(w, p["n_layers"], p["n_heads"], p["n_kv_heads"])
        elif "token_embd.weight" in w:  # llama.cpp naming (a .gguf file)
            from .gguf import convert_from_gguf
            w = convert_from_gguf(w, p["n_layers"])
            w.pop("rope_freqs.weight", None)
        w = {k: np.asarray(v).astype(np.float16) for k, v in w.items()}
        if self.quantize == "int8":
            w = Int8Linear.quantize(w, quantize_embeds=self.quantize_embeds)
        elif self.quantize == "nf4":
            w = self.linear.quantize(w)
        shards = self.model._shards
        if shards:
            if "output.weight" not in w:  # tied: the output layer is a window of the embedding table
                w["output.weight"] = w["tok_embeddings.weight"]
                if "tok_embeddings.scale" in w:
                    w["output.scale"] = w["tok_embeddings.scale"]
            for k, sh in shards.items():
                if k not in w:
                    continue
                w[k] = (w[k][sh.row0:sh.row0 + sh.rows] if k.endswith(".scale")
                        else w[k][sh.row0:sh.row0 + sh.rows, sh.col0:sh.col0 + sh.cols])
        load_state_dict(self.model, {k: np.ascontiguousarray(v) for k, v in w.items()}, strict=False)
        return self

    def load_synthetic(self, seed: int = synth.BASE_SEED) -> "Llama3":
        synth.fill_model(self.model, seed)
        return self

    # ---- generation
    def reset(self) -> None:
        self.start_pos, self.last_seen_toks = 0, []

    def _prefill(self, toks, batched: bool = False) -> Tensor | None:
        """Llama3._prefill (jsgrad/models/llama3.ts:298-312).  toks: a list of ids (one conversation) or int32 [B, n].
        At start_pos 0 the part of the prompt that equals what this object saw last is skipped — its K/V rows are
        still in the cache — exactly under the reference's rule: only when one of the two token lists is a prefix of
        the other.  The rest is fed one position per call as the reference does, or, with `batched`, in one
        multi-position forward.  Returns the token picked after the last position fed (None if nothing was fed)."""
        arr = np.asarray(toks, dtype=np.int32)
        if arr.ndim == 1:
            arr = arr[None, :]
        if self.start_pos == 0 and arr.shape[0] == 1:
            cur, last = arr[0].tolist(), list(self.last_seen_toks)
            n = min(len(cur), len(last))
            i = n if cur[:n] == last[:n] else 0
            self.start_pos += i
            self.last_seen_toks = cur
            arr = arr[:, i:]
        out = None
        if arr.shape[1] == 0:
            return out
        if batched:
            out = self.model.forward(arr, self.start_pos, self.temperature, self.top_k, self.top_p, self.alpha_f, self.alpha_p)
            self.start_pos += arr.shape[1]
            return out
        for i in range(arr.shape[1]):
            out = self.model.call(arr[:, i:i + 1], self.start_pos, self.temperature, self.top_k, self.top_p, self.alpha_f, self.alpha_p)
            self.start_pos += 1
        return out

    def _call(self, tok: int) -> int:
        """One token in, the sampled next token out (Llama3._call, jsgrad/models/llama3.ts:334-337)."""
        res = self.model.call(np.array([[tok]], np.int32), self.start_pos, self.temperature, self.top_k, self.top_p,
                              self.alpha_f, self.alpha_p)
        return int(res.numpy()[0])

    def _system(self, msg: str = "You are an helpful assistant.") -> None:
        """Llama3._system (jsgrad/models/llama3.ts:266-269): begin-of-text + the system turn go through the model."""
        if self.tokenizer is None:
            raise ValueError("no tokenizer: pass tokenizer=Tokenizer.llama(path) (the vocabulary file is not bundled)")
        self._prefill([self.tokenizer.bos_id, *self.tokenizer.encode_message("system", msg)], batched=True)

    def chat(self, messages: list[dict], on_token=None, max_tokens: int | None = None) -> dict:
        """Llama3.chat (jsgrad/models/llama3.ts:270-297): frame the turns, prefill all but the last prompt token, then
        feed tokens back one by one until a stop token comes out.  Returns {'message', 'stop_reason', 'usage'}.  The
        reference loops until a stop token; `max_tokens` and the context length bound the loop here
        (stop_reason 'max_tokens' / 'max_context')."""
        if self.tokenizer is None:
            raise ValueError("no tokenizer: pass tokenizer=Tokenizer.llama(path) (the vocabulary file is not bundled)")
        tk = self.tokenizer
        toks = [t for m in messages for t in tk.encode_message(m["role"], m["content"])] + tk.encode_role("assistant")
        st = time.perf_counter()
        self._prefill(toks[:-1], batched=True)
        usage = Llama3Usage(input_tokens=len(toks) - 1, time_to_first_token=time.perf_counter() - st)
        last_tok, message = toks[-1], {"role": "assistant", "content": ""}
        st = time.perf_counter()
        while True:
            if self.start_pos + 1 > self.max_context:
                return {"message": message, "stop_reason": "max_context", "usage": usage}
            tok = self._call(last_tok)
            self.start_pos += 1
            usage.output_tokens += 1
            usage.tokens_per_second = usage.output_tokens / max(time.perf_counter() - st, 1e-9)
            last_tok = tok
            if tok in tk.stop_tokens:
                return {"message": message, "stop_reason": "end_turn", "usage": usage}
            token = tk.decode([tok])
            message["content"] += token
            if on_token is not None:
                on_token({"message": message, "usage": usage, "token": token})
            if max_tokens is not None and usage.output_tokens >= max_tokens:
                return {"message": message, "stop_reason": "max_tokens", "usage": usage}

    def prefill(self, toks: np.ndarray) -> Tensor:
        """The whole prompt in one multi-position forward (Transformer.forward with S > 1, jsgrad/models/llama.ts:
        201-213) instead of one call per token; returns the greedy token after the last prompt position."""
        out = self.model.forward(np.asarray(toks, dtype=np.int32), self.start_pos, self.temperature, self.top_k, self.top_p,
                                 self.alpha_f, self.alpha_p)
        self.start_pos += toks.shape[1]
        return out

    def generate(self, prompt: np.ndarray, max_new_tokens: int) -> np.ndarray:
        """Greedy continuation through the public per-token API: every step copies the token ids to the device, runs
        the (graph-replayed) step and reads the chosen ids back — the `.item()` round trip of the reference's chat
        loop (jsgrad/models/llama3.ts:284-295,334-337).  prompt: int32 [B, n] -> int32 [B, max_new_tokens]."""
        if self.temperature >= 1e-6:
            raise ValueError("generate() is the greedy loop of the benchmark workloads: construct with temperature=0 "
                             "(sampling runs through chat() / _call())")
        prompt = np.asarray(prompt, dtype=np.int32)
        if prompt.ndim == 1:
            prompt = prompt[None, :]
        B = prompt.shape[0]
        st = time.perf_counter()
        self.last_seen_toks = []  # a seeded workload prompt is always fed whole
        tok = self._prefill(prompt).numpy()
        self.usage.time_to_first_token = time.perf_counter() - st
        out = np.empty((B, max_new_tokens), np.int32)
        st = time.perf_counter()
        for i in range(max_new_tokens):
            out[:, i] = tok
            if i + 1 < max_new_tokens:
                tok = self.model.call_host(tok.reshape(B, 1), self.start_pos)
                self.start_pos += 1
        self.usage.input_tokens, self.usage.output_tokens = int(prompt.size), int(out.size)
        self.usage.tokens_per_second = out.size / max(time.perf_counter() - st, 1e-9)
        return out
