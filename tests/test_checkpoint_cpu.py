"""Checkpoint conversion and the world tokenizer on the CPU: key translation and shape inference against the
reference's converter (where its checkout is present), round trip through the upstream layout, loading into this
package's model class; the tokenizer's greedy longest-match against the reference's trie on a synthetic vocabulary."""
import os
import random
import sys

import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from hf_adapter_b200.checkpoint import _template_shapes

REFERENCE = "/root/reference"
CFG = dict(vocab_size=64, hidden_size=128, num_hidden_layers=3, num_heads=2, head_dim=64, intermediate_size=256,
           decay_low_rank_dim=8, a_low_rank_dim=16, v_low_rank_dim=24, gate_low_rank_dim=32)


def _reference(module):
    if not os.path.isdir(os.path.join(REFERENCE, "rwkv7_hf")):
        pytest.skip("the reference checkout is not on this machine")
    sys.path.insert(0, REFERENCE)
    try:
        return __import__(f"rwkv7_hf.{module}", fromlist=["_"])
    finally:
        sys.path.remove(REFERENCE)


def _random_state_dict(seed=0):
    g = torch.Generator().manual_seed(seed)
    return {k: torch.randn(shape, generator=g) for k, shape in _template_shapes(hb.NativeRWKV7Config(**CFG)).items()}


def _upstream(sd):
    up = hb.to_upstream_state_dict(sd)
    # what official checkpoints look like: unused layer-0 value-gate factors, vectors with extra singleton axes
    up["blocks.0.att.v0"] = torch.zeros(128)
    up["blocks.0.att.v1"] = torch.zeros(128, 24)
    up["blocks.0.att.v2"] = torch.zeros(24, 128)
    up["blocks.1.att.r_k"] = up["blocks.1.att.r_k"].reshape(1, 2, 64)
    up["blocks.2.att.x_r"] = up["blocks.2.att.x_r"].reshape(128)
    return up


def test_template_shapes_are_the_model_state_dict():
    model = hb.RWKV7ForCausalLM(hb.NativeRWKV7Config(**CFG))
    assert {k: tuple(v.shape) for k, v in model.state_dict().items()} == _template_shapes(model.config)


def test_round_trip_and_load():
    sd = _random_state_dict()
    up = _upstream(sd)
    assert up["blocks.1.att.w1"].shape == (128, 8) and up["blocks.1.att.w2"].shape == (8, 128) and up["blocks.1.att.w0"].shape == (128,)
    assert "head.weight" in up and "blocks.0.ln0.weight" in up and "blocks.2.att.ln_x.bias" in up and "blocks.1.ffn.x_k" in up
    config, back = hb.convert_state_dict(up)
    assert (config.num_hidden_layers, config.hidden_size, config.num_heads, config.head_dim, config.intermediate_size,
            config.vocab_size) == (3, 128, 2, 64, 256, 64)
    assert (config.decay_low_rank_dim, config.a_low_rank_dim, config.v_low_rank_dim, config.gate_low_rank_dim) == (8, 16, 24, 32)
    assert set(back) == set(sd)
    for k in sd:
        assert back[k].shape == sd[k].shape and torch.equal(back[k], sd[k]), k
        assert back[k].data_ptr() != up.get(k, sd[k]).data_ptr()
    half = hb.convert_state_dict(up, dtype=torch.float16)[1]
    assert all(v.dtype == torch.float16 for v in half.values())
    model = hb.RWKV7ForCausalLM(config)
    model.load_state_dict(back)  # strict
    # a checkpoint with a hole, a gap in the block indices, a wrong projection shape
    broken = dict(up)
    del broken["blocks.1.att.a2"]
    with pytest.raises(KeyError, match="lacks tensors"):
        hb.convert_state_dict(broken)
    gap = {k.replace("blocks.2.", "blocks.3."): v for k, v in up.items()}
    with pytest.raises(ValueError, match="contiguous"):
        hb.convert_state_dict(gap)
    bad = dict(up)
    bad["blocks.1.att.key.weight"] = torch.zeros(64, 128)
    with pytest.raises(ValueError, match="expected"):
        hb.convert_state_dict(bad)
    with pytest.raises(KeyError, match="Unexpected"):
        hb.translate_name("optimizer.state", 3)


def test_translation_and_inference_match_the_reference_converter():
    conv = _reference("converter")
    up = _upstream(_random_state_dict(1))
    for name in up:
        assert hb.translate_name(name, 3) == conv.translate_name(name, 3), name
    ref_cfg = conv.infer_config(up, "float16", "chunk", False)
    cfg = hb.infer_config(up)
    for field in ("vocab_size", "hidden_size", "num_hidden_layers", "num_heads", "head_dim", "intermediate_size",
                  "decay_low_rank_dim", "a_low_rank_dim", "v_low_rank_dim", "gate_low_rank_dim"):
        assert getattr(cfg, field) == getattr(ref_cfg, field), field
    # the converted dict loads, strictly, into the reference's own model class
    ref_model = conv.build_template_model(ref_cfg, torch.float32)
    _, sd = hb.convert_state_dict(up)
    missing, unexpected = ref_model.load_state_dict(sd, strict=False)
    assert not missing and not unexpected


def _vocab(path):
    rng = random.Random(0)
    tokens = {i + 1: bytes([i]) for i in range(256)}  # every single byte: any input can be encoded
    words = ["the", "then", "there", "th", " a", " an", " and", "and", "\n\n", "  ", "    ", "é", "été", "日本", "日本語", "語",
             "🙂", "🙂🙂", "0", "00", "000", "=", "==", "==="]
    nxt = 300
    for w in words:
        tokens[nxt] = w.encode("utf-8")
        nxt += 1
    for _ in range(200):
        tokens[nxt] = bytes(rng.randrange(256) for _ in range(rng.randrange(2, 6)))
        nxt += 3  # gaps: ids without an entry
    tok = hb.RWKVWorldTokenizer(tokens=tokens)
    tok.save_vocabulary(path)
    return tokens


def test_tokenizer_longest_match_round_trip_and_file_format(tmp_path):
    path = str(tmp_path / "vocab.txt")
    tokens = _vocab(path)
    tok = hb.RWKVWorldTokenizer(path)
    assert tok.vocab_size == max(tokens) + 1 and tok.bytes_to_id == {v: k for k, v in tokens.items()}
    ids = tok.encode("then there was 日本語 and === 0000 🙂🙂🙂")
    by = tok.id_to_bytes
    assert [by[i] for i in ids[:3]] == [b"then", b" ", b"there"]
    assert b"".join(by[i] for i in ids).decode() == "then there was 日本語 and === 0000 🙂🙂🙂"
    assert tok.bytes_to_id["日本語".encode()] in ids and tok.bytes_to_id[b"==="] in ids and tok.bytes_to_id[b"000"] in ids
    rng = random.Random(1)
    for _ in range(200):
        raw = bytes(rng.randrange(256) for _ in range(rng.randrange(0, 40)))
        assert tok.decode_bytes(tok.encode_bytes(raw)) == raw
    assert tok.decode([10 ** 6, -1, 299]) == ""  # unknown ids and ids without an entry decode to nothing
    batch = tok(["the", "then there"], return_tensors="np")
    assert batch["input_ids"].shape == batch["attention_mask"].shape and batch["attention_mask"][0].tolist()[-1] == 1
    assert batch["attention_mask"][0, 0] == 0 and batch["input_ids"][0, 0] == 0
    no_bytes = hb.RWKVWorldTokenizer(tokens={1: b"a"})
    with pytest.raises(ValueError, match="cannot encode"):
        no_bytes.encode("ab")


def test_tokenizer_matches_the_reference_trie(tmp_path):
    ref = _reference("tokenization_rwkv7")
    path = str(tmp_path / "vocab.txt")
    _vocab(path)
    mine, theirs = hb.RWKVWorldTokenizer(path), ref._RWKVTrie(path)
    rng = random.Random(2)
    pieces = ["the", "n", " there", "日本語", "本", "🙂", "=", "0", " an", "d", "é", "t", "\n", " "]
    for _ in range(300):
        text = "".join(rng.choice(pieces) for _ in range(rng.randrange(0, 30)))
        ids = mine.encode(text)
        assert ids == theirs.encode(text)
        assert mine.decode(ids) == theirs.decode(ids) == text
    for _ in range(100):
        raw = bytes(rng.randrange(256) for _ in range(rng.randrange(1, 60)))
        assert mine.encode_bytes(raw) == theirs.encode_bytes(raw)
