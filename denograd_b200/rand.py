"""The random stream behind jsgrad's ``Tensor.rand`` (threefry2x32 counters, jsgrad/tensor.ts:773-843 and
jsgrad/ops.ts:1874-1890), restated on the host with numpy so that the stochastic branch of ``sample`` can be fed the
uniform samples the reference engine would draw: ``manual_seed(s)`` then one ``rand(n)`` per ``Tensor.rand`` call.

Per device the reference keeps a seed pair (sha256 of the number of devices seen before this one, taken modulo 2**32,
and ``Tensor._seed``) and a counter.  The first call on a device starts at counter 0; every later call first adds its
OWN word count to the counter (jsgrad/tensor.ts:820) and then draws.  A call for `num` float32 values draws
ceil(num/2) 64-bit threefry outputs: word i is the low half of block i, word ceil(num/2)+i its high half.
"""
from __future__ import annotations

import hashlib

import numpy as np

_ROT = ((13, 15, 26, 6), (17, 29, 16, 24))


def threefry2x32(x0: np.ndarray, x1: np.ndarray, key0: int, key1: int) -> tuple[np.ndarray, np.ndarray]:
    """Threefry-2x32, 20 rounds, on uint32 arrays (x0 = low word of the counter, x1 = high word)."""
    x0 = x0.astype(np.uint32).copy()
    x1 = x1.astype(np.uint32).copy()
    ks = (np.uint32(key1), np.uint32(key0 ^ key1 ^ 0x1BD11BDA), np.uint32(key0))
    with np.errstate(over="ignore"):
        x0 += ks[2]
        x1 += ks[0]
        for i in range(5):
            for r in _ROT[i % 2]:
                x0 += x1
                x1 = x0 ^ ((x1 << np.uint32(r)) | (x1 >> np.uint32(32 - r)))
            x0 += ks[i % 3]
            x1 += ks[(i + 1) % 3] + np.uint32(i + 1)
    return x0, x1


class DeviceRand:
    """Seed pair and counter of one device name, as ``Tensor._device_seeds`` / ``_device_rng_counters`` hold them."""

    def __init__(self, seed: int = 0, device_index: int = 0):
        digest = hashlib.sha256(int(device_index).to_bytes(4, "big", signed=True)).digest()
        self.seed0 = int.from_bytes(digest, "big") % (1 << 32)  # first entry of the pair
        self.seed1 = seed & 0xFFFFFFFF                           # Tensor._seed
        self.counter = 0
        self.fresh = True

    def rand(self, numel: int) -> np.ndarray:
        """float32 [numel] uniform in [0, 1), the values of one ``Tensor.rand([numel])`` call."""
        num = int(numel)
        if num == 0:
            return np.zeros((0,), np.float32)
        if self.fresh:
            self.fresh = False
        else:
            self.counter = (self.counter + num) & 0xFFFFFFFF
        half = (num + 1) // 2
        with np.errstate(over="ignore"):
            c0 = (np.arange(half, dtype=np.uint64) + np.uint64(self.counter)).astype(np.uint32)
            c1 = c0 + np.uint32(half & 0xFFFFFFFF)
        lo, hi = threefry2x32(c0, c1, self.seed0, self.seed1)
        bits = np.concatenate([lo, hi])[:num]
        # mantissa from the top 23 bits, exponent of 1.0, minus 1 (jsgrad/tensor.ts:828-836)
        f = ((bits >> np.uint32(9)) | np.uint32(0x3F800000)).view(np.float32)
        return (f - np.float32(1.0)).astype(np.float32)


_streams: dict[str, DeviceRand] = {}
_seed = 0


def manual_seed(seed: int = 0) -> None:
    """Tensor.manual_seed (jsgrad/tensor.ts:773-775): forget every device's seed pair and counter."""
    global _seed
    _seed = seed
    _streams.clear()


def rand(numel: int, device: str = "CUDA") -> np.ndarray:
    """Tensor.rand([numel]) on `device`: the n-th distinct device name seen since the last manual_seed gets the hash of
    n as the first word of its seed pair."""
    if device not in _streams:
        _streams[device] = DeviceRand(_seed, len(_streams))
    return _streams[device].rand(numel)
