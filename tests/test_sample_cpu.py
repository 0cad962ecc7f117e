"""CPU checks of the sampling restatements: the checker's `sample` / threefry (oracle/sample_oracle.c) against known
answers, and the package's numpy threefry stream (denograd_b200/rand.py) against the checker's C one."""
import numpy as np

from denograd_b200 import rand
from oracle import oracle as O


def test_threefry_known_answers():
    """Threefry-2x32 with 20 rounds: the published known-answer vectors of the Random123 library (counter, key ->
    output): zeros, all ones, and the digits of pi."""
    L = O.lib()
    kat = [((0x00000000, 0x00000000), (0x00000000, 0x00000000), (0x6b200159, 0x99ba4efe)),
           ((0xffffffff, 0xffffffff), (0xffffffff, 0xffffffff), (0x1cb996fc, 0xbb002be7)),
           ((0x243f6a88, 0x85a308d3), (0x13198a2e, 0x03707344), (0xc4923a9c, 0x483df7a0))]
    for (c0, c1), (k0, k1), (r0, r1) in kat:
        r = L.orc_threefry2x32(c0 | (c1 << 32), k0 | (k1 << 32))
        assert (r & 0xFFFFFFFF, r >> 32) == (r0, r1)
        a, b = rand.threefry2x32(np.array([c0], np.uint32), np.array([c1], np.uint32), k0, k1)
        assert (int(a[0]), int(b[0])) == (r0, r1)


def test_rand_stream_counter_rule_and_range():
    """The first call on a device starts at counter 0; each later call first advances the counter by its own word
    count (jsgrad/tensor.ts:820), then draws; values lie in [0, 1) with 23 random mantissa bits."""
    d = rand.DeviceRand(seed=4, device_index=0)
    a, b, c = d.rand(7), d.rand(5), d.rand(1000)
    assert (a == O.threefry_rand(d.seed0, 4, 0, 7)).all()
    assert (b == O.threefry_rand(d.seed0, 4, 5, 5)).all()
    assert (c == O.threefry_rand(d.seed0, 4, 1005, 1000)).all()
    assert c.dtype == np.float32 and (c >= 0).all() and (c < 1).all() and abs(float(c.mean()) - 0.5) < 0.05
    rand.manual_seed(4)
    assert (rand.rand(7, "CUDA") == a).all()
    assert not (rand.rand(7, "CUDA:1")[:5] == b).all()  # a second device name hashes to another seed word


def test_reference_order_sum():
    """Below 32768 elements a sum is one ascending pass; from there on, the largest divisor in [8, 256] splits it."""
    rng = np.random.default_rng(0)
    x = (rng.random(1000, dtype=np.float32) * 1e-3).astype(np.float32)
    s = np.float32(0)
    for v in x:
        s = np.float32(s + v)
    assert O.sum_f32(x) == float(s)
    n = 128256  # = 256 * 501
    x = (rng.random(n, dtype=np.float32) * 1e-5).astype(np.float32)
    parts = []
    for c in range(256):
        s = np.float32(0)
        for v in x[c * 501:(c + 1) * 501]:
            s = np.float32(s + v)
        parts.append(s)
    t = np.float32(0)
    for p in parts:
        t = np.float32(t + p)
    assert O.sum_f32(x) == float(t)


def test_sample_known_cases():
    rng = np.random.default_rng(3)
    lg = (rng.standard_normal(500) * 2).astype(np.float16).astype(np.float32)
    am = int(lg.argmax())
    assert O.sample(lg, 0.0, 0, 0.0, 0, 0, 0.7) == am            # greedy branch
    assert O.sample(lg, 0.9, 1, 1.0, 0, 0, 0.0) == am            # top-1 with p = 1 (threshold 0): only the maximum survives
    assert O.sample(lg, 0.9, 1, 1.0, 0, 0, 0.999) in (am, 0)     # u at the very top: an index past the end gathers 0
    # k = 0: the draw walks the cumulative distribution — u = 0 gives the first token with non-zero mass
    assert O.sample(lg, 0.9, 0, 0.0, 0, 0, 0.0) == 0
    # tie at the top: the lowest index wins the first round
    tie = lg.copy(); tie[40] = tie[7] = lg.max() + 1
    assert O.sample(tie, 0.5, 2, 1.0, 0, 0, 0.0) == 7
    # monotone in u
    picks = [O.sample(lg, 1.0, 0, 0.0, 0, 0, u) for u in np.linspace(0, 0.999, 50)]
    assert picks == sorted(picks)
    # alpha: the frequency penalty lowers a token that keeps being chosen; the counter counts
    cnt = np.zeros(500, np.int32)
    seq = [O.sample(lg, 0.05, 5, 1.0, 3.0, 0.0, 0.5, cnt) for _ in range(4)]
    assert cnt.sum() == 4 and len(set(seq)) > 1
