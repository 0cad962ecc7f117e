"""The reference's own hot-path test inputs (test/models/llama.test.ts:24-99: Llama-3.2-1B architecture built after
Tensor.manual_seed(4), one token at a given start position over an empty cache, temperature 0.85) run through the CUDA
path and the CPU checker.  The reference's expected output is not in its tree, so this pins nothing against the
reference: it shows that both sides, fed the reference's own seeded weights (narrowed to fp16), agree with each other,
and records what they produce (`-s` prints it)."""
import numpy as np
import pytest

from denograd_b200.device import Tensor
from denograd_b200.llama import sample
from denograd_b200.llama3 import Llama3
from oracle import oracle as O
from tests import reference_inputs as R

pytestmark = pytest.mark.gpu


def test_reference_test_inputs_agree_between_device_and_checker():
    sd, u = R.state_dict(4)
    p = dict(R.ARCH)
    llm = Llama3(size="1B", args=p, max_context=64, tied_output=False, temperature=R.TEMPERATURE).load_state_dict(sd)
    cfg = O.OracleConfig(dim=p["dim"], n_layers=p["n_layers"], n_heads=p["n_heads"], n_kv_heads=p["n_kv_heads"], hidden=p["hidden_dim"],
                         vocab=p["vocab_size"], max_context=64, max_batch=1, eps=p["norm_eps"], theta=float(p["rope_theta"]))
    ids = {"attention.wq": O.WQ, "attention.wk": O.WK, "attention.wv": O.WV, "attention.wo": O.WO,
           "feed_forward.w1": O.W1, "feed_forward.w2": O.W2, "feed_forward.w3": O.W3}
    for tok, start_pos in R.CALLS:
        m = O.OracleModel(cfg)  # a fresh (zero) cache per case, as each case of the reference test builds a new model
        for l in range(p["n_layers"]):
            for suffix, wid in ids.items():
                m.set_weight(l, wid, sd[f"layers.{l}.{suffix}.weight"])
            m.set_weight(l, O.ATTN_NORM, sd["norm.weight"]); m.set_weight(l, O.FFN_NORM, sd["norm.weight"])
        m.set_weight(-1, O.TOK_EMB, sd["tok_embeddings.weight"]); m.set_weight(-1, O.OUTPUT, sd["output.weight"])
        m.set_weight(-1, O.NORM, sd["norm.weight"])
        ref_logits, ref_greedy = m.forward(np.array([[tok]], np.int32), start_pos)
        m.close()
        llm.reset()
        dev = llm.model.dev
        llm.model.new_cache()  # empty cache: earlier cases must not leak into this one
        llm.model.forward(np.array([[tok]], np.int32), start_pos, 0.0)
        logits = llm.model.last_logits(1)
        dl = float(np.abs(logits - ref_logits).max())
        assert dl <= 2e-2, dl
        ut = Tensor(np.array([u], np.float32), device=dev)
        got = int(sample(llm.model._workspace(1).logits, R.TEMPERATURE, 0, 0.0, 0.0, 0.0, u=ut).numpy()[0])
        want_same_logits = O.sample(logits[0], R.TEMPERATURE, 0, 0.0, 0.0, 0.0, u)
        want = O.sample(ref_logits[0], R.TEMPERATURE, 0, 0.0, 0.0, 0.0, u)
        assert got == want_same_logits  # the sampler is exact given the logits
        top2 = np.sort(ref_logits[0])[-2:]
        print(f"reference test input (token {tok}, start_pos {start_pos}): greedy {int(ref_greedy[0])}, sampled at T=0.85 with "
              f"u={u:.7f}: device {got}, checker {want}; top-2 logit margin {top2[1] - top2[0]:.4f}; max |dlogit| {dl:.2e}")
