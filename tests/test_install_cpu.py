"""The rebinding a maintainer of the reference would do (hf_adapter_b200.install), applied to the reference's own
modules where its checkout is present: every operator name is replaced in the facade and in the decode / prefill /
recurrence modules it feeds, each replacement accepts the reference function's parameters by the same names and in
the same positional order, and uninstall restores the originals.  Plus the host-side pieces of the Hugging Face
surface that need no GPU: the cache's legacy form and counters, the mask contract, the sampler."""
import inspect
import os
import sys

import pytest
import torch

import hf_adapter_b200 as hb

REFERENCE = "/root/reference"


@pytest.fixture(scope="module")
def native_jit():
    if not os.path.isdir(os.path.join(REFERENCE, "rwkv7_hf")):
        pytest.skip("the reference checkout is not on this machine")
    sys.path.insert(0, REFERENCE)
    try:
        import rwkv7_hf.native_jit as nj
    finally:
        sys.path.remove(REFERENCE)
    return nj


def test_install_rebinds_reference_operator_names(native_jit):
    from rwkv7_hf import native_jit_decode, native_jit_prefill, native_jit_recurrent
    saved = hb.install(native_jit)
    try:
        assert len(saved) >= 20
        for name in saved:
            assert getattr(native_jit, name) is getattr(hb, name)
        assert native_jit_decode.fused_recurrent_output_prepare_raw is hb.fused_recurrent_output_prepare_raw
        assert native_jit_decode.fused_attn_norm_mix6_decode is hb.fused_attn_norm_mix6_decode
        assert native_jit_decode.fused_wavg_lora is hb.fused_wavg_lora
        assert native_jit_prefill.fused_recurrent_scan is hb.fused_recurrent_scan
        assert native_jit_prefill.self_chunk_rwkv7 is hb.self_chunk_rwkv7
        assert native_jit_prefill.fused_prefill_state_prep is hb.fused_prefill_state_prep
        assert native_jit_recurrent.fused_recurrent_update is hb.fused_recurrent_update
    finally:
        hb.uninstall(saved, native_jit)
    for name, original in saved.items():
        assert getattr(native_jit, name) is original
    assert native_jit_decode.fused_recurrent_output_prepare_raw is saved["fused_recurrent_output_prepare_raw"]


def test_replacements_take_the_reference_parameters(native_jit):
    POSITIONAL = (inspect.Parameter.POSITIONAL_ONLY, inspect.Parameter.POSITIONAL_OR_KEYWORD)
    checked = 0
    for name in hb.install.__globals__["OPERATOR_NAMES"]:
        if not hasattr(native_jit, name):
            continue
        ref = inspect.signature(inspect.unwrap(getattr(native_jit, name))).parameters
        own = inspect.signature(getattr(hb, name)).parameters
        ref_pos = [n for n, p in ref.items() if p.kind in POSITIONAL]
        own_pos = [n for n, p in own.items() if p.kind in POSITIONAL]
        assert own_pos[:len(ref_pos)] == ref_pos, f"{name}: positional parameters {own_pos} vs reference {ref_pos}"
        for n, p in ref.items():
            if p.kind == inspect.Parameter.KEYWORD_ONLY:
                assert n in own, f"{name}: keyword {n} of the reference is not accepted"
        for n, p in own.items():  # what this library adds must be optional
            if n not in ref and p.kind not in (inspect.Parameter.VAR_KEYWORD, inspect.Parameter.VAR_POSITIONAL):
                assert p.default is not inspect.Parameter.empty, f"{name}: extra parameter {n} has no default"
        checked += 1
    assert checked >= 20


def test_pack_tuple_matches_reference_layout(native_jit):
    """Slot by slot: the reference's extract_graph_packs on its own (CPU, random-init) model and this library's on a
    model loaded from the same state_dict give tensors of the same shapes in the same slots."""
    from rwkv7_hf import native_jit_packing
    from rwkv7_hf.model_config import NativeRWKV7Config as RefConfig
    from rwkv7_hf.native_model import NativeRWKV7ForCausalLM as RefModel
    torch.manual_seed(0)
    kw = dict(vocab_size=64, hidden_size=128, num_hidden_layers=2, num_heads=2, head_dim=64, intermediate_size=256,
              decay_low_rank_dim=8, a_low_rank_dim=8, v_low_rank_dim=8, gate_low_rank_dim=16)
    ref = RefModel(RefConfig(**kw)).eval()
    own = hb.RWKV7ForCausalLM(hb.NativeRWKV7Config(**kw))
    missing, unexpected = own.load_state_dict(ref.state_dict(), strict=False)
    assert not missing and not unexpected
    dense = lambda m: m.weight if isinstance(m, torch.nn.Linear) else m
    ref_packs, H, N, eps = native_jit_packing.extract_graph_packs(
        ref, rkv_policy="vkwr_auto", sparse_ffn_low_memory_pack_enabled=lambda: False,
        try_relayout_ffn_value_weight=lambda m: None, graph_linear_operand=dense,
        graph_linear_is_dense=lambda o: isinstance(o, torch.Tensor))
    own_packs, H2, N2, eps2 = hb.extract_graph_packs(own, rkv_policy="vkwr_auto")
    assert (H, N, eps) == (H2, N2, eps2) and len(ref_packs) == len(own_packs)
    for rp, op in zip(ref_packs, own_packs):
        assert len(rp) == len(op) == 41
        for slot, (a, b) in enumerate(zip(rp, op)):
            if isinstance(a, torch.Tensor):
                assert isinstance(b, torch.Tensor) and a.shape == b.shape, f"slot {slot}: {tuple(a.shape)} vs {getattr(b, 'shape', b)}"
                assert torch.equal(a, b), f"slot {slot}"
            else:
                assert a == b, f"slot {slot}"
    state, xpa, xpf = hb.init_batched_from_packs(own_packs, 3, "cpu", torch.float32)
    ref_state, ref_xpa, ref_xpf = native_jit_packing.init_batched_from_packs(ref_packs, 3, "cpu", torch.float32)
    assert [t.shape for t in state] == [t.shape for t in ref_state] and [t.shape for t in xpa] == [t.shape for t in ref_xpa]


def test_legacy_cache_round_trip_and_counters():
    c = hb.NativeRWKV7Cache.allocate(2, 3, 128, 2, 64, "cpu", torch.float16)
    c.seen_tokens = 7
    legacy = c.to_legacy_cache()
    assert isinstance(legacy, tuple) and len(legacy) == 4 and legacy.get_seq_length() == 7 and legacy.to_legacy_cache() is legacy
    back = hb.NativeRWKV7Cache.from_legacy_cache(legacy)
    assert back.get_seq_length() == 7 and back[0][0] is c[0][0]
    assert hb.NativeRWKV7Cache.from_legacy_cache(()).get_batch_size() is None
    with pytest.raises(TypeError):
        hb.NativeRWKV7Cache.from_legacy_cache((1, 2, 3))
    d = c.clone()
    d.select_batch(torch.tensor([2, 0]))
    d.reorder_cache(torch.tensor([1, 0]))
    d.batch_repeat_interleave(2)
    d.crop(0)
    m = d.rwkv7_cache_metrics()
    assert (m["clones"], m["select_batch_calls"], m["reorder_calls"], m["batch_repeat_interleave_calls"], m["crops"], m["resets"]) == (1, 2, 1, 1, 1, 1)
    assert m["batch_size"] == 4 and m["layers"] == 2 and m["seen_tokens"] == 0
    assert c.rwkv7_cache_metrics()["clones"] == 0


def test_attention_mask_contract():
    from hf_adapter_b200.model import _validate_attention_mask
    assert _validate_attention_mask(None, 2, 3) is None
    assert _validate_attention_mask(torch.ones(2, 3), 2, 3) is None
    m = _validate_attention_mask(torch.tensor([[0, 1, 1], [1, 1, 1]]), 2, 3)
    assert m.dtype == torch.bool and m.tolist() == [[False, True, True], [True, True, True]]
    with pytest.raises(ValueError):
        _validate_attention_mask(torch.ones(2, 5), 2, 3)
    cut = _validate_attention_mask(torch.tensor([[0, 0, 1, 0, 1]]), 1, 2, allow_trailing=True)
    assert cut.tolist() == [[False, True]]
    with pytest.raises(TypeError):
        _validate_attention_mask([[1, 1]], 1, 2)


def test_sampler_respects_top_k_top_p_and_seed():
    torch.manual_seed(0)
    logits = torch.randn(5, 50)
    assert torch.equal(hb.sample_next_token(logits, temperature=0.0), logits.argmax(-1))
    g = lambda: torch.Generator().manual_seed(3)
    a = hb.sample_next_token(logits, temperature=0.8, top_k=5, generator=g())
    b = hb.sample_next_token(logits, temperature=0.8, top_k=5, generator=g())
    assert torch.equal(a, b)
    top5 = logits.topk(5, -1).indices
    for _ in range(20):
        t = hb.sample_next_token(logits, top_k=5)
        assert all(int(t[i]) in top5[i].tolist() for i in range(5))
    assert torch.equal(hb.sample_next_token(logits, top_p=1e-6), logits.argmax(-1))  # only the most likely token survives
    p = torch.softmax(logits, -1)
    sp, si = p.sort(-1, descending=True)
    nucleus = [set(si[i, : int((sp[i].cumsum(0) - sp[i] < 0.5).sum())].tolist()) for i in range(5)]
    for _ in range(20):
        t = hb.sample_next_token(logits, top_p=0.5)
        assert all(int(t[i]) in nucleus[i] for i in range(5))
