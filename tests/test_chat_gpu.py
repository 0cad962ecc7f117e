"""The chat driver on the GPU (Llama3._system / chat / _prefill, jsgrad/models/llama3.ts:266-312) with a synthetic
vocabulary: framing, prefix reuse, stop tokens, usage accounting, and the stochastic path end to end."""
import numpy as np
import pytest

from denograd_b200 import rand
from denograd_b200.llama3 import Llama3
from denograd_b200.tokenizer import LLAMA3_PATTERN, Tokenizer, llama3_special_tokens
from oracle import oracle as O
from tests.golden.gen_golden import TINY
from tests.test_tokenizer import _ranks
from tests.util import build_oracle

pytestmark = pytest.mark.gpu


def _tok():
    r = _ranks()
    return Tokenizer(LLAMA3_PATTERN, r, llama3_special_tokens(len(r)))


def test_greedy_chat_matches_the_checker_and_reuses_the_prefix():
    tk = _tok()
    llm = Llama3(size="1B", args=TINY, max_context=256, tied_output=True, temperature=0, tokenizer=tk).load_synthetic()
    llm._system("hello world")
    n_sys = llm.start_pos
    assert n_sys == 1 + len(tk.encode_message("system", "hello world"))
    msgs = [{"role": "user", "content": "the world 123"}]
    seen = []
    res = llm.chat(msgs, on_token=lambda r: seen.append(r["token"]), max_tokens=6)
    toks = [t for m in msgs for t in tk.encode_message(m["role"], m["content"])] + tk.encode_role("assistant")
    assert res["usage"].input_tokens == len(toks) - 1 and 1 <= res["usage"].output_tokens <= 6
    assert res["stop_reason"] in ("end_turn", "max_tokens") and res["message"]["content"] == "".join(seen)
    # the checker, token by token over the same framed prompt
    m = build_oracle(TINY, max_context=256, max_batch=1, int8=False, tied=True)
    full = [tk.bos_id, *tk.encode_message("system", "hello world"), *toks]
    pos, nxt = 0, None
    for t in full:
        _, nxt = m.forward(np.array([[t]], np.int32), pos); pos += 1
    want = []
    for _ in range(res["usage"].output_tokens):
        want.append(int(nxt[0]))
        if want[-1] in tk.stop_tokens:
            break
        _, nxt = m.forward(np.array([[want[-1]]], np.int32), pos); pos += 1
    got_text = tk.decode([t for t in want if t not in tk.stop_tokens])
    assert res["message"]["content"] == got_text
    # prefix reuse: after a reset the same leading tokens are skipped, only the new tail is fed
    end_pos = llm.start_pos
    llm.start_pos = 0
    llm.last_seen_toks = full[:20]
    llm._prefill(full[:25])
    assert llm.start_pos == 25 and llm.last_seen_toks == full[:25]
    llm.start_pos = 0
    llm._prefill([full[0] + 1] + full[1:10])  # differs at the first token: nothing is reused
    assert llm.start_pos == 10
    assert end_pos > n_sys


def test_sampled_chat_is_reproducible_and_follows_sample():
    tk = _tok()
    kw = dict(size="1B", args=TINY, max_context=128, tied_output=True, tokenizer=tk, top_k=8, top_p=0.9, temperature=0.8)
    outs = []
    for _ in range(2):
        rand.manual_seed(7)
        llm = Llama3(**kw).load_synthetic()
        res = llm.chat([{"role": "user", "content": "hello"}], max_tokens=5)
        outs.append(res["message"]["content"])
    assert outs[0] == outs[1]
    # one step by hand: the token the kernel picks equals the checker's `sample` on the very logits the device produced
    rand.manual_seed(3)
    llm = Llama3(**kw).load_synthetic()
    llm._prefill([1, 2, 3], batched=True)
    tok = llm._call(5)
    logits = llm.model.last_logits(1)[0]
    rand.manual_seed(3)
    us = rand.rand(1, llm.model.dev.device), rand.rand(1, llm.model.dev.device)  # the prefill's pick drew the first one
    assert tok == O.sample(logits, 0.8, 8, 0.9, 0.0, 0.0, float(us[1][0]))
