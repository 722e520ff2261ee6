"""The Hugging Face surface (forward with attention_mask / inputs_embeds / caches, generate, sampling) and the
pack-tuple layer step, on the GPU.  Masked forward passes are checked against a fixture the reference produced
(tests/golden/model_masked.npz: same tiny fp32 weights as model_tiny.npz)."""
import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from tests.gpu_util import cu, golden, npf
from tests.test_model_gpu import load_tiny, tiny_cfg

pytestmark = pytest.mark.gpu


def test_masked_forward_matches_reference_fixture():
    model = load_tiny(golden("model_tiny.npz"))
    g = golden("model_masked.npz")
    ids, mask = cu(g["ids"]), cu(g["mask"])
    out = model(ids, attention_mask=mask, use_cache=True)
    assert type(out).__name__ == "CausalLMOutputWithPast"
    np.testing.assert_allclose(npf(out.logits), g["logits"], rtol=3e-4, atol=3e-4)
    cache = out.past_key_values
    st, xpa, xpf, vf = cache
    np.testing.assert_allclose(npf(torch.stack(st)), g["state"], rtol=3e-4, atol=3e-5)
    np.testing.assert_allclose(npf(torch.stack(xpa)), g["xpa"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(npf(torch.stack(xpf)), g["xpf"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(npf(vf), g["v_first"], rtol=2e-4, atol=2e-5)
    assert cache.get_seq_length() == int(g["seen"])
    # the same through embeddings
    emb = model.model.embeddings(ids)
    oe = model(inputs_embeds=emb, attention_mask=mask)
    np.testing.assert_allclose(npf(oe.logits), g["embeds_logits"], rtol=3e-4, atol=3e-4)
    # cached continuation with the full-length mask (its last columns are used)
    o2 = model(cu(g["more"]), attention_mask=cu(g["mask2"]), past_key_values=cache)
    np.testing.assert_allclose(npf(o2.logits), g["more_logits"], rtol=3e-4, atol=3e-4)
    np.testing.assert_allclose(npf(torch.stack(o2.past_key_values[0])), g["more_state"], rtol=3e-4, atol=3e-5)
    assert o2.past_key_values.get_seq_length() == int(g["more_seen"])


def test_left_padded_rows_equal_unpadded_sequences():
    """A masked prefix leaves a row where a shorter, unpadded prompt would (fp32 model; the two runs go through
    different kernels -- decode steps against the layer-wise prefill -- so equality is up to fp32 rounding)."""
    model = load_tiny(golden("model_tiny.npz"))
    torch.manual_seed(3)
    ids = torch.randint(0, 256, (2, 6), device="cuda")
    mask = torch.tensor([[0, 0, 1, 1, 1, 1], [1, 1, 1, 1, 1, 1]], device="cuda")
    both = model(ids, attention_mask=mask, logits_to_keep=1)
    alone = model(ids[:1, 2:], logits_to_keep=1)
    assert both.logits.shape == (2, 1, 256)
    torch.testing.assert_close(both.logits[0], alone.logits[0], rtol=2e-4, atol=2e-4)
    for a, b in zip(both.past_key_values[0], alone.past_key_values[0]):
        torch.testing.assert_close(a[:1], b, rtol=2e-4, atol=2e-5)
    gen = model.generate(ids, attention_mask=mask, max_new_tokens=3)
    gen_alone = model.generate(ids[:1, 2:], max_new_tokens=3)
    assert torch.equal(gen[0, 6:], gen_alone[0, 4:])


def test_forward_argument_validation_and_tuple_outputs():
    model = load_tiny(golden("model_tiny.npz"))
    ids = torch.randint(0, 256, (2, 5), device="cuda")
    with pytest.raises(ValueError, match="either input_ids or inputs_embeds"):
        model(ids, inputs_embeds=torch.zeros(2, 5, 128, device="cuda"))
    with pytest.raises(ValueError, match="requires input_ids or inputs_embeds"):
        model()
    with pytest.raises(ValueError, match="last dimension must match hidden_size"):
        model(inputs_embeds=torch.zeros(2, 5, 64, device="cuda"))
    with pytest.raises(ValueError, match="attention_mask must have the same"):
        model(ids, attention_mask=torch.ones(2, 4, device="cuda"))
    with pytest.raises(NotImplementedError):
        model(ids, output_attentions=True)
    logits, cache = model(ids, return_dict=False)
    assert logits.shape == (2, 5, 256) and isinstance(cache, hb.NativeRWKV7Cache)
    with pytest.raises(ValueError, match="batch size"):
        model(ids[:1, :1], past_key_values=cache)
    (only_logits,) = model(ids, return_dict=False, use_cache=False)
    assert torch.equal(only_logits, logits)
    legacy = model(ids, return_legacy_cache=True).past_key_values
    assert isinstance(legacy, tuple) and legacy.get_seq_length() == 5
    nxt = model(ids[:, :1], past_key_values=legacy)  # a legacy tuple in gives a legacy tuple out
    assert isinstance(nxt.past_key_values, tuple) and nxt.past_key_values.get_seq_length() == 6
    inputs = model.prepare_inputs_for_generation(torch.cat([ids, ids[:, :1]], 1), past_key_values=cache,
                                                 attention_mask=torch.ones(2, 6, device="cuda"))
    assert inputs["input_ids"].shape == (2, 1) and inputs["attention_mask"].shape == (2, 1) and inputs["use_cache"] is True
    first = model.prepare_inputs_for_generation(ids, attention_mask=torch.ones(2, 5, device="cuda"))
    assert first["input_ids"].shape == (2, 5) and first["past_key_values"] is None
    re = model._reorder_cache(cache, torch.tensor([1, 0], device="cuda"))
    assert re.rwkv7_cache_metrics()["select_batch_calls"] == 1


def test_generate_sampling_and_eos():
    model = load_tiny(golden("model_tiny.npz"))
    ids = cu(golden("model_tiny.npz")["ids"])
    greedy = model.generate(ids, max_new_tokens=5)
    gen = lambda seed: torch.Generator(device="cuda").manual_seed(seed)
    a = model.generate(ids, max_new_tokens=5, do_sample=True, temperature=0.9, top_k=20, top_p=0.9, generator=gen(1))
    b = model.generate(ids, max_new_tokens=5, do_sample=True, temperature=0.9, top_k=20, top_p=0.9, generator=gen(1))
    assert torch.equal(a, b) and a.shape == greedy.shape
    one = model.generate(ids, max_new_tokens=5, do_sample=True, top_k=1)  # top-1 sampling is greedy
    assert torch.equal(one, greedy)
    eos = int(greedy[0, ids.shape[1] + 1])  # row 0 emits this as its second new token
    stopped = model.generate(ids, max_new_tokens=5, eos_token_id=eos, pad_token_id=0)
    T = ids.shape[1]
    assert int(stopped[0, T + 1]) == eos and bool((stopped[0, T + 2:] == 0).all())
    row1_stop = (greedy[1, T:] == eos).nonzero()
    upto = int(row1_stop[0]) + 1 if len(row1_stop) else stopped.shape[1] - T
    assert torch.equal(stopped[1, T:T + upto], greedy[1, T:T + upto])


def test_pack_step_runs_a_dense_and_a_quantised_model():
    """block_ip_batched from packs == the model's own decode step (which is that loop), for dense weights, where the
    projection slots hold tensors and slot 40 the stacked r/k/v, and for int4 projections, where they hold modules."""
    torch.manual_seed(5)
    cfg = hb.NativeRWKV7Config(vocab_size=256, hidden_size=256, num_hidden_layers=3, num_heads=4, head_dim=64,
                               intermediate_size=512, decay_low_rank_dim=16, a_low_rank_dim=16, v_low_rank_dim=8,
                               gate_low_rank_dim=32)
    model = hb.RWKV7ForCausalLM(cfg)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(0.2 * torch.randn_like(p))
    model = model.half().cuda().eval()
    for quant in (None, "mm4"):
        if quant:
            hb.quantize_model(model, quant, min_params=1)
        packs, H, N, eps = hb.extract_graph_packs(model, rkv_policy="vkwr_auto")
        assert len(packs) == 3 and all(len(p) == 41 for p in packs) and (H, N) == (4, 64)
        if quant:
            assert isinstance(packs[0][20], hb.MM4Linear) and packs[0][40].numel() == 0
        else:
            assert hb.graph_linear_is_dense(packs[0][20]) and packs[0][40].shape == (3, 256, 256)
        assert packs[0][4] == 1 and packs[1][4] == 0 and packs[0][30].shape == (1, 256) and packs[0][31].shape == (256, 1)
        ids = torch.randint(0, 256, (5,), device="cuda")
        cache = model.new_cache(5)
        for _ in range(2):
            want = model.rwkv7_forward_token(ids, cache, use_graph=False)
        state, xpa, xpf = hb.init_batched_from_packs(packs, 5, "cuda", torch.float16)
        v_first = torch.zeros(5, 256, device="cuda", dtype=torch.float16)
        for _ in range(2):
            x = model.model.embeddings(ids)
            x, state, xpa, xpf, v_first = hb.step_batched(model, x, state, xpa, xpf, v_first, packs)
        got = model.lm_head(torch.nn.functional.layer_norm(x, (256,), model.model.norm.weight, model.model.norm.bias))
        torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-3)
        for a, b in zip(state, cache[0]):
            assert torch.equal(a, b)
        assert torch.equal(v_first, cache[3])
    with pytest.raises(ValueError, match="41 slots"):
        hb.block_ip_batched(x, state[0], xpa[0], xpf[0], v_first, packs[0][:40])


def test_speculative_generate_equals_target_greedy():
    """Whatever the draft proposes, the result is the target's greedy continuation: a draft that always agrees (the
    target itself), one that rarely does (other random weights), block sizes that do and do not divide the length."""
    g = golden("model_tiny.npz")
    target = load_tiny(g)
    ids = cu(g["ids"])[:1]
    want = target.generate(ids, max_new_tokens=11)
    same = target.rwkv7_speculative_generate(ids, target, max_new_tokens=11, draft_tokens=4, return_stats=True)
    assert torch.equal(same["sequences"], want)
    st = same["stats"]
    assert st["acceptance_rate"] == 1.0 and st["corrected_tokens"] == 0 and st["generated_tokens"] == 11 and st["resyncs"] == 0
    assert st["target_forward_calls"] == 1 + 3  # prompt + three verified blocks (4 + 4 + 3)
    torch.manual_seed(9)
    other = hb.RWKV7ForCausalLM(tiny_cfg())
    with torch.no_grad():
        for p in other.parameters():
            p.copy_(0.3 * torch.randn_like(p))
    other = other.cuda().eval()
    for block in (1, 3, 5):
        res = target.rwkv7_speculative_generate(ids, other, max_new_tokens=11, draft_tokens=block, return_stats=True)
        assert torch.equal(res["sequences"], want), block
        st = res["stats"]
        assert st["accepted_tokens"] + st["corrected_tokens"] == 11 and st["proposed_tokens"] >= st["accepted_tokens"]
        assert st["resync_tokens"] <= st["resyncs"] * block
    eos = int(want[0, ids.shape[1] + 2])
    stopped = target.rwkv7_speculative_generate(ids, other, max_new_tokens=11, draft_tokens=3, eos_token_id=eos)
    first = int((want[0, ids.shape[1]:] == eos).nonzero()[0])
    assert torch.equal(stopped, want[:, :ids.shape[1] + first + 1])
    with pytest.raises(ValueError):
        target.rwkv7_speculative_generate(cu(g["ids"]), other)  # batch of two
    assert torch.equal(target.rwkv7_speculative_generate(ids, other, max_new_tokens=0), ids)


def test_prefill_graph_replays_equal_eager_prefill():
    g = golden("model_tiny.npz")
    model = load_tiny(g)
    torch.manual_seed(4)
    ids = torch.randint(0, 256, (2, 24), device="cuda")
    want_logits, want_cache = model.rwkv7_prefill_chunks(ids, None, chunk_size=8)
    runner = hb.PrefillGraph(model, 2, 8)
    cache = None
    for t0 in range(0, 24, 8):
        logits, cache = runner.replay(ids[:, t0:t0 + 8], cache)
    torch.testing.assert_close(logits, want_logits, rtol=1e-5, atol=1e-5)
    for a, b in zip(cache._tensors(), want_cache._tensors()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    assert cache.get_seq_length() == 24
    # another cache through the same graph, interleaved with the first
    other_logits, other = runner.replay(ids[:, :8].flip(0), None)
    more, cache = runner.replay(ids[:, :8], cache)
    ref_logits, ref = model.rwkv7_prefill_native(ids[:, :8].flip(0), None)
    torch.testing.assert_close(other_logits, ref_logits, rtol=1e-5, atol=1e-5)
    ref_more, want_cache = model.rwkv7_prefill_native(ids[:, :8], want_cache)
    torch.testing.assert_close(more, ref_more, rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        runner.replay(ids[:, :4], None)


def test_checkpoint_to_tokens_end_to_end():
    """Upstream-layout weights -> load_checkpoint (fp16, int4 projections) -> tokenizer batch with left padding ->
    generate: the padded row continues exactly as the same prompt alone."""
    g = golden("model_tiny.npz")
    sd = {k[len("param::"):]: torch.from_numpy(v) for k, v in g.items() if k.startswith("param::")}
    upstream = hb.to_upstream_state_dict(sd)
    model = hb.load_checkpoint(upstream, dtype=torch.float16, quant="mm4", min_params=1)
    assert isinstance(model.model.layers[0].attn.r_proj, hb.MM4Linear) and model.dtype == torch.float16
    tokens = {i + 1: bytes([i]) for i in range(200)}
    tokens.update({210: b"the", 211: b" state", 212: b" machine"})
    tok = hb.RWKVWorldTokenizer(tokens=tokens)
    batch = tok(["the state", "the state machine runs"], device="cuda")
    assert batch["attention_mask"][0, 0] == 0 and batch["input_ids"].shape[0] == 2
    out = model.generate(batch["input_ids"], attention_mask=batch["attention_mask"], max_new_tokens=4)
    alone = tok(["the state"], device="cuda")
    out_alone = model.generate(alone["input_ids"], max_new_tokens=4)
    assert torch.equal(out[0, -4:], out_alone[0, -4:])
    assert isinstance(tok.decode(out[1].tolist()), str)
