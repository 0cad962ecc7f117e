"""GGUF container and ggml block dequantisation (denograd_b200/gguf.py) against element-by-element restatements of the
published ggml block formats, on a file written by this test."""
import struct

import numpy as np
import pytest

from denograd_b200.gguf import convert_from_gguf, ggml_data_to_tensor, gguf_load


def f16bytes(x) -> bytes:
    return np.float16(x).tobytes()


# ---- writers: quantise `vals` into ggml blocks (quality does not matter, only that every bit field is exercised)
def q4_0(vals):
    out = b""
    for blk in vals.reshape(-1, 32):
        d = np.float16(np.abs(blk).max() / 7 + 1e-3)
        q = np.clip(np.round(blk / np.float32(d)) + 8, 0, 15).astype(np.uint8)
        out += f16bytes(d) + bytes(q[:16] | (q[16:] << 4))
    return out


def q4_1(vals):
    out = b""
    for blk in vals.reshape(-1, 32):
        m = np.float16(blk.min()); d = np.float16((blk.max() - blk.min()) / 15 + 1e-3)
        q = np.clip(np.round((blk - np.float32(m)) / np.float32(d)), 0, 15).astype(np.uint8)
        out += f16bytes(d) + f16bytes(m) + bytes(q[:16] | (q[16:] << 4))
    return out


def q8_0(vals):
    out = b""
    for blk in vals.reshape(-1, 32):
        d = np.float16(np.abs(blk).max() / 127 + 1e-4)
        out += f16bytes(d) + np.clip(np.round(blk / np.float32(d)), -127, 127).astype(np.int8).tobytes()
    return out


def q6_k(rng, n_blocks):
    """Random but fully populated Q6_K blocks: returns (bytes, expected float32 values by the ggml formula)."""
    out, want = b"", []
    for _ in range(n_blocks):
        ql = rng.integers(0, 256, 128, dtype=np.uint8)
        qh = rng.integers(0, 256, 64, dtype=np.uint8)
        sc = rng.integers(-60, 61, 16).astype(np.int8)
        d = np.float16(rng.uniform(1e-3, 3e-3))
        out += ql.tobytes() + qh.tobytes() + sc.tobytes() + f16bytes(d)
        y = np.zeros(256, np.float32)
        df = np.float32(d)
        for half in range(2):  # dequantize_row_q6_K of ggml, written out per element
            L, H, S = ql[half * 64:], qh[half * 32:], sc[half * 8:]
            for l in range(32):
                i = l // 16
                q1 = int((L[l] & 0xF) | (((H[l] >> 0) & 3) << 4)) - 32
                q2 = int((L[l + 32] & 0xF) | (((H[l] >> 2) & 3) << 4)) - 32
                q3 = int((L[l] >> 4) | (((H[l] >> 4) & 3) << 4)) - 32
                q4 = int((L[l + 32] >> 4) | (((H[l] >> 6) & 3) << 4)) - 32
                for off, q, s in ((0, q1, S[i]), (32, q2, S[i + 2]), (64, q3, S[i + 4]), (96, q4, S[i + 6])):
                    y[half * 128 + l + off] = np.float32(np.float32(df * np.float32(q)) * np.float32(s))
        want.append(y)
    return out, np.concatenate(want)


def test_block_formats_element_by_element():
    rng = np.random.default_rng(0)
    vals = rng.standard_normal(128).astype(np.float32)
    raw = np.frombuffer(q4_0(vals), np.uint8)
    got = ggml_data_to_tensor(raw, 128, 2)
    want = []
    for b in range(4):
        blk = raw[b * 18:(b + 1) * 18]
        d = np.float32(blk[:2].view(np.float16)[0])
        qs = blk[2:]
        want += [np.float32((int(qs[j] & 0xF) - 8)) * d for j in range(16)] + [np.float32((int(qs[j] >> 4) - 8)) * d for j in range(16)]
    assert (got == np.array(want, np.float32)).all() and np.abs(got - vals).max() < 0.4
    raw = np.frombuffer(q4_1(vals), np.uint8)
    got = ggml_data_to_tensor(raw, 128, 3)
    want = []
    for b in range(4):
        blk = raw[b * 20:(b + 1) * 20]
        d, m = np.float32(blk[:2].view(np.float16)[0]), np.float32(blk[2:4].view(np.float16)[0])
        qs = blk[4:]
        want += [np.float32(np.float32(int(qs[j] & 0xF)) * d + m) for j in range(16)] + [np.float32(np.float32(int(qs[j] >> 4)) * d + m) for j in range(16)]
    assert (got == np.array(want, np.float32)).all() and np.abs(got - vals).max() < 0.3
    raw = np.frombuffer(q8_0(vals), np.uint8)
    got = ggml_data_to_tensor(raw, 128, 8)
    want = []
    for b in range(4):
        blk = raw[b * 34:(b + 1) * 34]
        d = np.float32(blk[:2].view(np.float16)[0])
        want += [d * np.float32(q) for q in blk[2:].view(np.int8)]
    assert (got == np.array(want, np.float32)).all() and np.abs(got - vals).max() < 0.03
    blob, want = q6_k(rng, 3)
    got = ggml_data_to_tensor(np.frombuffer(blob, np.uint8), 768, 14)
    assert (got == want).all()
    for typ, dt in ((0, np.float32), (1, np.float16), (16, np.int8), (17, np.int16), (18, np.int32)):
        a = (rng.standard_normal(10) * 50).astype(dt)
        assert (ggml_data_to_tensor(np.frombuffer(a.tobytes(), np.uint8), 10, typ) == a).all()
    with pytest.raises(ValueError):
        ggml_data_to_tensor(raw, 32, 12)  # Q4_K: not among the reference's formats


def _s(x: str) -> bytes:
    return struct.pack("<Q", len(x.encode())) + x.encode()


def write_gguf(path, kv, tensors, align=32):
    """tensors: list of (name, dims innermost-first, ggml type, payload bytes)."""
    head = b"GGUF" + struct.pack("<iqq", 3, len(tensors), len(kv))
    for k, (tag, v) in kv.items():
        head += _s(k) + struct.pack("<i", tag)
        if tag == 8:
            head += _s(v)
        elif tag == 9:
            inner, items = v
            head += struct.pack("<iQ", inner, len(items)) + b"".join(_s(i) if inner == 8 else struct.pack("<i", i) for i in items)
        else:
            head += struct.pack({4: "<I", 5: "<i", 6: "<f", 10: "<Q"}[tag], v)
    body, off = b"", 0
    for name, dims, typ, payload in tensors:
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<iQ", typ, off)
        pad = -len(payload) % align
        body += payload + b"\0" * pad
        off += len(payload) + pad
    head += b"\0" * (-len(head) % align)
    with open(path, "wb") as f:
        f.write(head + body)


def test_container_round_trip_and_key_map(tmp_path):
    rng = np.random.default_rng(1)
    emb = rng.standard_normal((64, 32)).astype(np.float32)           # [vocab 64][dim 32]
    wq = rng.standard_normal((32, 32)).astype(np.float32)
    norm = np.ones(32, np.float32)
    blob6, want6 = q6_k(rng, 8)                                       # 2048 values = [64][32]
    path = tmp_path / "tiny.gguf"
    write_gguf(path, {"general.architecture": (8, "llama"), "general.alignment": (4, 64), "llama.block_count": (4, 1),
                      "tokenizer.ggml.tokens": (9, (8, ["a", "b", "c"])), "some.ints": (9, (5, [1, -2, 3]))},
               [("token_embd.weight", [32, 64], 14, blob6), ("blk.0.attn_q.weight", [32, 32], 8, q8_0(wq.reshape(-1))),
                ("blk.0.attn_norm.weight", [32], 0, norm.tobytes()), ("output_norm.weight", [32], 0, norm.tobytes()),
                ("blk.0.ffn_gate.weight", [32, 64], 1, emb.astype(np.float16).tobytes())], align=64)
    kv, sd = gguf_load(open(path, "rb").read())
    assert kv["general.architecture"] == "llama" and kv["tokenizer.ggml.tokens"] == ["a", "b", "c"] and kv["some.ints"] == [1, -2, 3]
    assert sd["token_embd.weight"].shape == (64, 32) and (sd["token_embd.weight"].reshape(-1) == want6).all()
    assert sd["blk.0.attn_q.weight"].shape == (32, 32) and np.abs(sd["blk.0.attn_q.weight"] - wq).max() < 0.05
    assert (sd["blk.0.ffn_gate.weight"] == emb.astype(np.float16)).all()
    m = convert_from_gguf(sd, 1)
    assert set(m) == {"tok_embeddings.weight", "output.weight", "layers.0.attention.wq.weight", "layers.0.attention_norm.weight",
                      "norm.weight", "layers.0.feed_forward.w1.weight"}
    assert m["output.weight"] is sd["token_embd.weight"]
    from denograd_b200.state import load_checkpoint
    assert (load_checkpoint(str(path))["output_norm.weight"] == norm).all()
    with pytest.raises(ValueError):
        gguf_load(b"GGUX" + open(path, "rb").read()[4:])
