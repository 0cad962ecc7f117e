"""CPU checks of the checkpoint reader: safetensors container round trip (incl. bf16 and a sharded index), and the
Hugging Face -> Llama conversion (names, q/k rotary row permutation)."""
import json
import os

import numpy as np
import pytest

from denograd_b200.state import (_permute, bf16_to_f16, convert_from_huggingface, load_checkpoint, safe_load, safe_save)


def test_safetensors_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    t = {"a.weight": rng.standard_normal((5, 7)).astype(np.float16), "b": rng.integers(-128, 127, (3, 4, 2)).astype(np.int8),
         "c": rng.standard_normal(9).astype(np.float32), "empty_dim": np.zeros((0, 4), np.float16)}
    fn = str(tmp_path / "x.safetensors")
    safe_save(t, fn, metadata={"format": "pt"})
    raw = open(fn, "rb").read()
    n = int.from_bytes(raw[:8], "little")
    assert n % 8 == 0 and json.loads(raw[8:8 + n])["__metadata__"] == {"format": "pt"}
    back = safe_load(fn)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and (back[k] == t[k]).all()


def test_bf16_is_narrowed_through_float32(tmp_path):
    x = np.array([1.0, -2.5, 3.140625, 65280.0, 1e-8, 70000.0], np.float32)
    bits = (x.view(np.uint32) >> 16).astype(np.uint16)  # truncation keeps these values exactly representable in bf16
    want = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float16)
    assert (bf16_to_f16(bits).view(np.uint16) == want.view(np.uint16)).all()
    # a file that declares BF16: written by hand, read back as float16
    header = json.dumps({"w": {"dtype": "BF16", "shape": [2, 3], "data_offsets": [0, 12]}}).encode()
    header += b" " * (-len(header) % 8)
    fn = tmp_path / "b.safetensors"
    fn.write_bytes(len(header).to_bytes(8, "little") + header + bits.tobytes())
    got = safe_load(str(fn))["w"]
    assert got.dtype == np.float16 and got.shape == (2, 3) and (got.reshape(-1).view(np.uint16) == want.view(np.uint16)).all()


def test_sharded_checkpoint_through_its_index(tmp_path):
    a = {"x": np.arange(6, dtype=np.float16).reshape(2, 3)}
    b = {"y": np.arange(4, dtype=np.float32), "z": np.ones((2, 2), np.int8)}
    safe_save(a, str(tmp_path / "m-1.safetensors"))
    safe_save(b, str(tmp_path / "m-2.safetensors"))
    idx = tmp_path / "model.safetensors.index.json"
    idx.write_text(json.dumps({"weight_map": {"x": "m-1.safetensors", "y": "m-2.safetensors", "z": "m-2.safetensors"}}))
    w = load_checkpoint(str(idx))
    assert set(w) == {"x", "y", "z"} and (w["x"] == a["x"]).all() and (w["y"] == b["y"]).all()
    with pytest.raises(ValueError):
        load_checkpoint(str(tmp_path / "model.bin"))  # neither safetensors, an index, nor gguf


def test_malformed_files_are_rejected(tmp_path):
    fn = tmp_path / "bad.safetensors"
    fn.write_bytes(b"\x00\x01")
    with pytest.raises(ValueError):
        safe_load(str(fn))
    fn.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(ValueError):
        safe_load(str(fn))
    header = json.dumps({"w": {"dtype": "F16", "shape": [4], "data_offsets": [0, 64]}}).encode()
    header += b" " * (-len(header) % 8)
    fn.write_bytes(len(header).to_bytes(8, "little") + header + b"\x00" * 8)
    with pytest.raises(ValueError):
        safe_load(str(fn))


def test_huggingface_names_and_rotary_row_permutation():
    L, H, G, hd, d, f, V = 2, 4, 2, 8, 32, 48, 64
    rng = np.random.default_rng(1)
    hf = {"model.embed_tokens.weight": rng.standard_normal((V, d)).astype(np.float16),
          "model.norm.weight": np.ones(d, np.float16), "lm_head.weight": rng.standard_normal((V, d)).astype(np.float16),
          "model.layers.0.self_attn.rotary_emb.inv_freq": np.ones(hd // 2, np.float32)}
    for l in range(L):
        hf[f"model.layers.{l}.input_layernorm.weight"] = np.full(d, l + 1, np.float16)
        hf[f"model.layers.{l}.post_attention_layernorm.weight"] = np.full(d, l + 2, np.float16)
        for x, rows in (("q", H * hd), ("k", G * hd), ("v", G * hd), ("o", d)):
            hf[f"model.layers.{l}.self_attn.{x}_proj.weight"] = rng.standard_normal((rows, d)).astype(np.float16)
        for x, shape in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f))):
            hf[f"model.layers.{l}.mlp.{x}_proj.weight"] = rng.standard_normal(shape).astype(np.float16)
    sd = convert_from_huggingface(hf, L, H, G)
    assert "layers.1.feed_forward.w1.weight" in sd and (sd["layers.1.feed_forward.w1.weight"] == hf["model.layers.1.mlp.gate_proj.weight"]).all()
    assert (sd["layers.0.feed_forward.w2.weight"] == hf["model.layers.0.mlp.down_proj.weight"]).all()
    assert (sd["layers.0.feed_forward.w3.weight"] == hf["model.layers.0.mlp.up_proj.weight"]).all()
    assert (sd["layers.0.attention.wv.weight"] == hf["model.layers.0.self_attn.v_proj.weight"]).all()  # v and o: untouched
    assert (sd["layers.1.ffn_norm.weight"] == 3).all() and (sd["output.weight"] == hf["lm_head.weight"]).all()
    assert not any("rotary_emb" in k for k in sd)
    # row j of head h in the Llama layout (pair i = j // 2, member m = j % 2) is Hugging Face row m * hd/2 + i of that head
    q_hf, q = hf["model.layers.0.self_attn.q_proj.weight"], sd["layers.0.attention.wq.weight"]
    for h in range(H):
        for j in range(hd):
            assert (q[h * hd + j] == q_hf[h * hd + (j % 2) * (hd // 2) + j // 2]).all()
    k_hf, k = hf["model.layers.1.self_attn.k_proj.weight"], sd["layers.1.attention.wk.weight"]
    assert (k == _permute(k_hf, G)).all() and not (k == k_hf).all()
    with pytest.raises(KeyError):
        convert_from_huggingface({"model.layers.0.mlp.router.weight": np.zeros((1, 1), np.float16)}, L, H, G)
