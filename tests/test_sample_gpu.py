"""GPU parity of the stochastic `sample` kernel (jg_sample) against the CPU checker's restatement of
jsgrad/models/llama.ts:131-185: the chosen token ids must be identical — the kernel adds its float32 sums in the
reference's own order, so there is no tolerance to state."""
import numpy as np
import pytest

from denograd_b200 import ffi, rand
from denograd_b200.device import Tensor
from denograd_b200.llama import sample
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _logits(rng, rows, V, spread):
    return (rng.standard_normal((rows, V)) * spread).astype(np.float16)


@pytest.mark.parametrize("V", [1000, 2048, 40000, 128256])
@pytest.mark.parametrize("k,p", [(0, 0.0), (1, 0.0), (40, 0.8), (40, 0.0), (7, 1.0), (200, 0.95)])
def test_sampled_ids_equal_the_checker(dev, V, k, p):
    rng = np.random.default_rng(V + 31 * k)
    rows = 3
    lg = _logits(rng, rows, V, 3.0)
    lg[1, 5] = lg[1, 900] = lg[1].max() + np.float16(1.0)  # a tie at the top: the lowest index must win a round
    lt = Tensor(lg, device=dev)
    out = Tensor.empty((rows,), "int32", dev)
    for temp in (0.95, 0.3):
        for trial in range(4):
            u = rng.random(rows, dtype=np.float32)
            dev.call("jg_sample", out.ptr, lt.ptr, Tensor(u, device=dev).ptr, 0, rows, V, temp, k, p, 0.0, 0.0)
            got = out.numpy()
            want = [O.sample(lg[r].astype(np.float32), temp, k, p, 0.0, 0.0, float(u[r])) for r in range(rows)]
            assert got.tolist() == want, (V, k, p, temp, trial)


def test_alpha_penalties_and_counter(dev):
    rng = np.random.default_rng(9)
    V, rows = 5000, 2
    lg = _logits(rng, rows, V, 2.0)
    lt = Tensor(lg, device=dev)
    cnt = Tensor.zeros((rows, V), "int32", dev)
    ref_cnt = np.zeros((rows, V), np.int32)
    out = Tensor.empty((rows,), "int32", dev)
    for step in range(12):  # a low temperature keeps picking the same few tokens: the penalties must move the pick on
        u = rng.random(rows, dtype=np.float32)
        dev.call("jg_sample", out.ptr, lt.ptr, Tensor(u, device=dev).ptr, cnt.ptr, rows, V, 0.2, 20, 0.9, 0.7, 0.4)
        want = [O.sample(lg[r].astype(np.float32), 0.2, 20, 0.9, 0.7, 0.4, float(u[r]), ref_cnt[r]) for r in range(rows)]
        assert out.numpy().tolist() == want, step
    assert (cnt.numpy() == ref_cnt).all() and ref_cnt.sum() == 24


def test_sample_wrapper_and_argument_checks(dev):
    rng = np.random.default_rng(2)
    V = 3000
    lg = _logits(rng, 1, V, 2.0)
    lt = Tensor(lg, device=dev)
    # temperature below 1e-6: argmax, lowest index among equals
    assert int(sample(lt, 0.0, 0, 0.0, 0.0, 0.0).numpy()[0]) == O.sample(lg[0].astype(np.float32), 0.0, 0, 0.0, 0, 0, 0.5)
    # default uniform source: the restated Tensor.rand stream
    rand.manual_seed(11)
    got = [int(sample(lt, 0.9, 0, 0.0, 0.0, 0.0).numpy()[0]) for _ in range(3)]
    rand.manual_seed(11)
    us = [float(rand.rand(1, dev.device)[0]) for _ in range(3)]
    assert got == [O.sample(lg[0].astype(np.float32), 0.9, 0, 0.0, 0, 0, u) for u in us]
    with pytest.raises(ValueError):
        sample(lt, 0.9, 0, 1.5, 0.0, 0.0)
    with pytest.raises(ValueError):
        sample(lt, 0.9, V + 1, 0.5, 0.0, 0.0)
    with pytest.raises(ffi.JgError):
        dev.call("jg_sample", lt.ptr, lt.ptr, lt.ptr, 0, 1, V, 0.9, 600, 0.5, 0.0, 0.0)  # k beyond the kernel's table
