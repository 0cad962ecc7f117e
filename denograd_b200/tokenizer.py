"""Llama-3 tokenizer — Python mirror of jsgrad/models/tokenizer.ts (byte-pair encoding over a tiktoken-style rank file,
the Llama-3 split pattern, the special-token table and the chat framing helpers).

The vocabulary file (``tokenizer.model``: one ``<base64 token> <rank>`` per line) is not shipped with this package
and cannot be downloaded here; ``Tokenizer.llama(path)`` reads one the caller has, and ``Tokenizer(...)`` takes any rank
table directly (the tests use a small synthetic one).  Same names, argument meaning and quirks as the reference:
``encode`` splits with the pattern and merges greedily by lowest rank (jsgrad/models/tokenizer.ts:55-103), ``decode``
drops ids outside the mergeable table (:42-53), ``encode_role`` / ``encode_message`` frame a chat turn (:104-109).
"""
from __future__ import annotations

import base64

import regex  # \\p{L}, \\p{N}: the standard library's `re` has no Unicode property classes

# jsgrad/models/tokenizer.ts:26 — flags 'giu': global matching is `finditer`, case-insensitive, Unicode.
LLAMA3_PATTERN = (r"'s|'t|'re|'ve|'m|'ll|'d|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
                  r"|\s+(?!\S)|\s+")


def llama3_special_tokens(n_ranks: int) -> dict[str, int]:
    """The special-token table exactly as the reference builds it (jsgrad/models/tokenizer.ts:10-30): ten named
    entries followed by 246 more whose names restart at `reserved_special_token_0` (the reference numbers them by the
    position in the mapped range, not by its value), ids n_ranks + position; a later duplicate name replaces the
    earlier id, as `Object.fromEntries` does."""
    names = ["<|begin_of_text|>", "<|end_of_text|>", "<|reserved_special_token_0|>", "<|reserved_special_token_1|>",
             "<|reserved_special_token_2|>", "<|reserved_special_token_3|>", "<|start_header_id|>", "<|end_header_id|>",
             "<|reserved_special_token_4|>", "<|eot_id|>"]
    names += [f"<|reserved_special_token_{i}|>" for i in range(len(range(5, 256 - 5)))]
    out: dict[str, int] = {}
    for i, name in enumerate(names):
        out[name] = n_ranks + i
    return out


class Tokenizer:
    def __init__(self, pat, mergeable_ranks: dict[bytes, int], special_tokens: dict[str, int]):
        """pat: compiled `regex` pattern (or its source); mergeable_ranks: token bytes -> rank (= id)."""
        self.pat = regex.compile(pat, regex.IGNORECASE | regex.UNICODE) if isinstance(pat, str) else pat
        self.mergeable_ranks = mergeable_ranks
        self.special_tokens = special_tokens
        self.decode_map = {i: tok for tok, i in mergeable_ranks.items()}

    @staticmethod
    def llama(path: str) -> "Tokenizer":
        """Tokenizer.llama (jsgrad/models/tokenizer.ts:6-31): parse `<base64> <rank>` lines."""
        ranks: dict[bytes, int] = {}
        with open(path, "r") as f:
            for line in f.read().split("\n"):
                if not line:
                    continue
                k, v = line.split(" ")[:2]
                ranks[base64.b64decode(k)] = int(v)
        return Tokenizer(LLAMA3_PATTERN, ranks, llama3_special_tokens(len(ranks)))

    @property
    def bos_id(self) -> int:
        return self.special_tokens["<|begin_of_text|>"]

    @property
    def stop_tokens(self) -> list[int]:
        return [self.special_tokens["<|end_of_text|>"], self.special_tokens["<|eot_id|>"]]

    def decode(self, toks: list[int]) -> str:
        """Concatenate the byte strings of the ids inside the mergeable table (special ids are dropped) and decode
        them as UTF-8 with replacement, like TextDecoder (jsgrad/models/tokenizer.ts:42-53)."""
        n = len(self.mergeable_ranks)
        return b"".join(self.decode_map[t] for t in toks if t < n).decode("utf-8", errors="replace")

    def encode(self, text: str, allow_special: bool = False) -> list[int]:
        tokens: list[int] = []
        for m in self.pat.finditer(text):
            piece = m.group(0)
            if allow_special and piece in self.special_tokens:
                tokens.append(self.special_tokens[piece])
            else:
                tokens.extend(self.bpe_encode(piece.encode("utf-8")))
        return tokens

    def bpe_encode(self, data: bytes) -> list[int]:
        """Greedy byte-pair merging (jsgrad/models/tokenizer.ts:67-103): repeatedly take the adjacent pair with the
        lowest rank (the first such pair on ties of position) and merge every occurrence of exactly that pair, left to
        right, until no adjacent pair is in the table."""
        parts = [bytes([b]) for b in data]
        ranks = self.mergeable_ranks
        while True:
            min_rank, merge = None, None
            for i in range(len(parts) - 1):
                r = ranks.get(parts[i] + parts[i + 1])
                if r is not None and (min_rank is None or r < min_rank):
                    min_rank, merge = r, (parts[i], parts[i + 1])
            if merge is None:
                break
            new, i = [], 0
            while i < len(parts):
                if i < len(parts) - 1 and parts[i] == merge[0] and parts[i + 1] == merge[1]:
                    new.append(parts[i] + parts[i + 1])
                    i += 2
                else:
                    new.append(parts[i])
                    i += 1
            parts = new
        return [ranks[p] for p in parts]

    def encode_role(self, role: str) -> list[int]:
        return [self.special_tokens["<|start_header_id|>"], *self.encode(role), self.special_tokens["<|end_header_id|>"],
                *self.encode("\n\n")]

    def encode_message(self, role: str, content: str) -> list[int]:
        return [*self.encode_role(role), *self.encode(content.strip()), self.special_tokens["<|eot_id|>"]]
