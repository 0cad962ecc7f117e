"""denograd_b200 — a B200-native `CUDA` device for jsgrad's Llama-3 forward (prefill + KV-cached greedy decode).

Layout:
  csrc/      hand-written sm_100a CUDA kernels and the C ABI (include/jsgrad_cuda.h) -> lib/libjsgrad_cuda.so
  ffi.py     ctypes binding of that ABI (the Python twin of ts/ops_cuda.ts's Deno.dlopen table)
  device.py  CUDA (Compiled), CUDAAllocator, Buffer, Tensor, CUDAGraph — jsgrad/device.ts + runtime/allocator.ts
  nn.py      Linear, Int8Linear, RMSNorm, Embedding, Int8Embedding, state dicts — jsgrad/nn + models/llama3.ts
  llama.py   Attention, FeedForward, TransformerBlock, Transformer, TinyJit — jsgrad/models/llama.ts
  llama3.py  MODEL_PARAMS, Llama3 (load, prefill, greedy generation) — jsgrad/models/llama3.ts
  synth.py   seeded synthetic weights / tokens for the benchmark workloads
  ts/        the TypeScript device that binds the same ABI from Deno
"""
from .device import CUDA, Buffer, CUDAGraph, Device, Tensor  # noqa: F401
