"""The decode step as one persistent kernel (jg_step_create / jg_step_run) against the CPU checker and against the
launch-per-op path of the same model: same ids away from ties, logits within the fp16 bar."""
import numpy as np
import pytest

from denograd_b200 import synth
from denograd_b200.llama3 import Llama3
from tests.test_llama_gpu import LOGIT_TOL, greedy_with_logits, make
from tests.util import build_oracle, oracle_greedy

pytestmark = pytest.mark.gpu

# a shape the kernel is instantiated for (head_dim 64, 4 query heads per kv head, hidden rows of 13 KB: two per 32 KB pass and four per 64 KB pass, as in the 1B model) with
# ragged row counts: 1003 vocabulary rows and 6656 hidden rows do not divide by the number of CTAs
SMALL = {"dim": 256, "n_heads": 4, "n_kv_heads": 1, "n_layers": 3, "norm_eps": 1e-5, "rope_theta": 500000,
         "vocab_size": 1003, "hidden_dim": 6656}


def safe_prefix(ids, ref_ids, ref_logits, margins, b):
    ulp = 2.0 ** (np.floor(np.log2(np.abs(ref_logits.max(axis=2)))) - 10)
    safe = (margins / ulp) >= 3
    n = ids.shape[1] if safe[:, b].all() else int(np.argmin(safe[:, b]))
    return n


@pytest.mark.parametrize("B", [1, 2])
def test_single_kernel_step_matches_checker(B):
    prompt = synth.prompt_tokens(9, SMALL["vocab_size"], batch=B, seed=77)
    llm = make("1B", args=SMALL, max_context=128, max_batch=2, tied_output=False)
    m = build_oracle(SMALL, max_context=128, max_batch=B, tied=False)
    ref_ids, ref_logits, margins = oracle_greedy(m, prompt, 10)
    ids, logits = greedy_with_logits(llm, prompt, 10)
    assert llm.model._single_kernel_step(B) is not None, "the model did not take the single-kernel step"
    assert np.abs(logits - ref_logits).max() <= LOGIT_TOL
    for b in range(B):
        n = safe_prefix(ids, ref_ids, ref_logits, margins, b)
        assert (ids[b, :n] == ref_ids[b, :n]).all(), (b, n)


def test_single_kernel_step_equals_launch_per_op_path(monkeypatch):
    B = 2
    prompt = synth.prompt_tokens(21, SMALL["vocab_size"], batch=B, seed=78)
    llm = make("1B", args=SMALL, max_context=128, max_batch=2, tied_output=True)
    ids, logits = greedy_with_logits(llm, prompt, 12)
    assert llm.model._single_kernel_step(B) is not None
    monkeypatch.setenv("JG_STEP_KERNEL", "0")
    ref = make("1B", args=SMALL, max_context=128, max_batch=2, tied_output=True)
    ids2, logits2 = greedy_with_logits(ref, prompt, 12)
    assert ref.model._single_kernel_step(B) is None
    assert np.abs(logits - logits2).max() <= 1e-2  # summation order only
    m = build_oracle(SMALL, max_context=128, max_batch=B, tied=True)
    ref_ids, ref_logits, margins = oracle_greedy(m, prompt, 12)
    for b in range(B):
        n = safe_prefix(ids, ref_ids, ref_logits, margins, b)
        assert (ids[b, :n] == ids2[b, :n]).all() and (ids[b, :n] == ref_ids[b, :n]).all()


def test_a_run_of_steps_in_one_launch_equals_step_by_step():
    """decode_loop hands the whole run to one launch (the kernel feeds its picks back itself); rows at different
    positions; the picks equal those of one launch per step."""
    B, n = 2, 16
    prompt = synth.prompt_tokens(14, SMALL["vocab_size"], batch=B, seed=79)
    llm = make("1B", args=SMALL, max_context=128, max_batch=2, tied_output=False)
    ids, _ = greedy_with_logits(llm, prompt, n + 1)      # step by step through call()
    llm2 = make("1B", args=SMALL, max_context=128, max_batch=2, tied_output=False)
    first = llm2._prefill(prompt).numpy()
    assert (first == ids[:, 0]).all()
    run = llm2.model.decode_loop(first, llm2.start_pos, n)
    assert run.shape == (B, n) and (run == ids[:, 1:]).all()
    # continuing on the device (tokens and positions were advanced by the kernel)
    more = llm2.model.decode_loop(first, llm2.start_pos + n, 4, resume=True)
    nxt = ids[:, -1]
    for i in range(4):
        nxt = llm.model.call(nxt.reshape(B, 1), llm.start_pos, 0.0).numpy()
        llm.start_pos += 1
        assert (more[:, i] == nxt).all(), i


def test_unsupported_shapes_keep_the_launch_per_op_path():
    from tests.golden.gen_golden import TINY  # two query heads per kv head: no instantiation
    llm = make("1B", args=TINY, max_context=64, max_batch=2, tied_output=True)
    prompt = synth.prompt_tokens(5, TINY["vocab_size"], batch=1, seed=3)
    greedy_with_logits(llm, prompt, 3)
    assert llm.model._single_kernel_step(1) is None

