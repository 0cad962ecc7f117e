"""The Llama-3 tokenizer mirror (denograd_b200/tokenizer.py) against small hand-checked cases and an independent
slow restatement of the reference's merge loop (jsgrad/models/tokenizer.ts:67-103).  The real vocabulary file is not
available here, so the rank table is synthetic: all 256 bytes plus a few merges."""
import base64

import pytest

from denograd_b200.tokenizer import LLAMA3_PATTERN, Tokenizer, llama3_special_tokens


def _ranks():
    r = {bytes([b]): b for b in range(256)}
    for i, tok in enumerate([b"he", b"ll", b"hell", b"lo", b"hello", b" w", b"or", b" wor", b"ld", b"\n\n", b" world", b"th", b"the", b"12", b"123"]):
        r[tok] = 256 + i
    return r


@pytest.fixture()
def tok():
    r = _ranks()
    return Tokenizer(LLAMA3_PATTERN, r, llama3_special_tokens(len(r)))


def slow_bpe(ranks, data: bytes):
    """Reference loop, written from its description: find the lowest-ranked adjacent pair, merge all its occurrences."""
    parts = [bytes([b]) for b in data]
    while True:
        best = None
        for i in range(len(parts) - 1):
            r = ranks.get(parts[i] + parts[i + 1])
            if r is not None and (best is None or r < best[0]):
                best = (r, parts[i], parts[i + 1])
        if best is None:
            return [ranks[p] for p in parts]
        out, i = [], 0
        while i < len(parts):
            if i + 1 < len(parts) and parts[i] == best[1] and parts[i + 1] == best[2]:
                out.append(parts[i] + parts[i + 1]); i += 2
            else:
                out.append(parts[i]); i += 1
        parts = out


def test_bpe_merges_by_lowest_rank(tok):
    r = tok.mergeable_ranks
    assert tok.encode("hello") == [r[b"hello"]]
    assert tok.encode("hello world") == [r[b"hello"], r[b" world"]]
    assert tok.encode("hell") == [r[b"hell"]]
    # "he" (rank 256) merges before "th" (267); "t" + "he" is then found as "the"
    assert tok.encode("the") == [r[b"the"]]
    assert tok.encode("tho") == [r[b"th"], ord("o")]
    for text in ("hello hello  world\n\nthe 12345 lo", "héllo wörld", "'s 're  \t\n x"):
        want = []
        for m in tok.pat.finditer(text):
            want += slow_bpe(r, m.group(0).encode())
        assert tok.encode(text) == want
        assert tok.decode(tok.encode(text)) == text


def test_split_pattern(tok):
    pieces = [m.group(0) for m in tok.pat.finditer("Hello, world!  It's 12345\n\nnew")]
    assert pieces == ["Hello", ",", " world", "!", " ", " It", "'s", " ", "123", "45", "\n\n", "new"]


def test_special_tokens_and_chat_framing(tok):
    n = len(tok.mergeable_ranks)
    st = tok.special_tokens
    assert tok.bos_id == n and tok.stop_tokens == [n + 1, n + 9]
    assert st["<|start_header_id|>"] == n + 6 and st["<|end_header_id|>"] == n + 7
    # the reference numbers the trailing reserved tokens from 0 again, so the later duplicates take over the names
    assert st["<|reserved_special_token_0|>"] == n + 10 and st["<|reserved_special_token_4|>"] == n + 14
    assert len(st) == 10 + 246 - 5 and max(st.values()) == n + 255
    role = tok.encode_role("user")
    assert role[0] == st["<|start_header_id|>"] and role[-1] == tok.mergeable_ranks[b"\n\n"]
    msg = tok.encode_message("user", "  hello world \n")
    assert msg[:len(role)] == role and msg[-1] == st["<|eot_id|>"]
    assert msg[len(role):-1] == tok.encode("hello world")
    assert tok.encode("<|eot_id|>") != [st["<|eot_id|>"]]          # specials are plain text unless allowed
    assert tok.decode([st["<|eot_id|>"], tok.mergeable_ranks[b"hello"]]) == "hello"  # special ids are dropped


def test_rank_file_round_trip(tmp_path):
    r = _ranks()
    path = tmp_path / "tokenizer.model"
    path.write_text("\n".join(f"{base64.b64encode(k).decode()} {v}" for k, v in r.items()) + "\n")
    t = Tokenizer.llama(str(path))
    assert t.mergeable_ranks == r and t.bos_id == len(r)
    assert t.encode("hello world") == [r[b"hello"], r[b" world"]]
