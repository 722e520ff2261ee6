"""GPU parity at the sizes the benchmark configurations state: the 0.1B-shape fp32 model against the reference's
greedy token stream (512-token prompt + 128 steps), the quantised projection operators at 4096 x 4096 / 4096 x 16384 /
16384 x 4096 with 1, 8 and 64 rows, the int8 GEMM at 4096 rows bit for bit, one 7.2B-width int4 layer against the
oracle, the fused A8W8 FFN against the reference's own composition, and ragged chunked scans."""
import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from oracle import rwkv7_oracle as O
from tests.golden.seeded_weights import checksum, seeded_state_dict
from tests.gpu_util import cu, golden, npf, rel_err, wkv_inputs
from tests.test_oracle_golden import params_from_golden

pytestmark = pytest.mark.gpu
N = 64


def test_config1_0p1b_fp32_prefill_and_128_greedy_steps_match_reference():
    """12 layers, d_model 768, 12 heads, FFN 3072, vocabulary 65536, LoRA ranks 64/64/32/128, fp32, batch 1: the
    reference's eager prefill of a 512-token prompt and its 128 cached greedy steps (fixture config1.npz; weights
    rebuilt from the same seeded recipe, checked by checksum).  Tokens identical, logits within 3e-4."""
    g = golden("config1.npz")
    cfg = hb.NativeRWKV7Config(vocab_size=65536, hidden_size=768, num_hidden_layers=12, num_heads=12, head_dim=64,
                               intermediate_size=3072, decay_low_rank_dim=64, a_low_rank_dim=64, v_low_rank_dim=32,
                               gate_low_rank_dim=128)
    model = hb.RWKV7ForCausalLM(cfg)
    sd = seeded_state_dict({k: v.shape for k, v in model.state_dict().items()}, int(g["weight_seed"]))
    np.testing.assert_allclose(checksum(sd), g["weights_checksum"], rtol=1e-12)
    model.load_state_dict(sd)
    model = model.float().cuda().eval()
    ids = cu(g["ids"])
    assert tuple(ids.shape) == (1, 512)
    out = model(ids, use_cache=True, logits_to_keep=1)
    logits, cache = out.logits[:, -1], out.past_key_values
    np.testing.assert_allclose(npf(logits), g["prefill_logits"], rtol=3e-4, atol=3e-4)
    toks = []
    for step in range(128):
        tok = logits.argmax(-1)
        toks.append(tok)
        logits = model.rwkv7_forward_token(tok, cache, use_graph=True)
    toks = torch.stack(toks, 1).cpu().numpy()
    assert float(g["top2_gap"].min()) > 1.5e-3  # no greedy step of the fixture is a near-tie (5x the logit tolerance)
    assert np.array_equal(toks, g["greedy"]), f"first mismatch at step {int(np.argmax(toks != g['greedy']))}"
    np.testing.assert_allclose(npf(logits), g["final_logits"], rtol=1e-3, atol=1e-3)
    assert cache.get_seq_length() == 512 + 128
    st, xpa, xpf, vf = cache
    np.testing.assert_allclose([float(s.double().norm()) for s in st], g["final_state_norm"], rtol=1e-3)
    np.testing.assert_allclose([float(s.double().norm()) for s in xpa], g["final_xpa_norm"], rtol=1e-3)
    np.testing.assert_allclose([float(s.double().norm()) for s in xpf], g["final_xpf_norm"], rtol=1e-3)
    np.testing.assert_allclose(npf(st[-1][0, 0]), g["final_state_l11_h0"], rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(npf(vf), g["final_v_first"], rtol=1e-3, atol=1e-3)


def _dequant_ref(x, Wq):
    """fp64 matmul against the dequantised fp16 weight: what the formats define."""
    return x.astype(np.float64) @ Wq.astype(np.float64).T


@pytest.mark.parametrize("K,Nout", [(4096, 4096), (4096, 16384), (16384, 4096)])
def test_config3_decode_projections_full_size(K, Nout):
    """Weights ~ N(0, 0.02), activations ~ N(0, 1) fp16, M in {1, 8, 64}: int4 group-128 (implicit zero-point 8 and a
    random zero-point variant) on the tensor-core kernel and on the CUDA-core GEMV, int8 per-output-channel on its
    GEMV, against the dequantised fp64 product (tolerance 2e-3 of the output scale)."""
    from hf_adapter_b200 import _lib
    rng = np.random.default_rng(K + Nout)
    W = (0.02 * rng.standard_normal((Nout, K))).astype(np.float16)
    packed, scales = O.quantize_w4_groupwise(W, 128)
    W4 = O.dequant_w4_groupwise(packed, scales)
    zr = rng.integers(5, 12, scales.shape, dtype=np.uint8)
    W4z = O.dequant_w4_groupwise(packed, scales, zr)
    q8, s8 = O.quantize_w8_row(W)
    W8 = (q8.astype(np.float32) * s8.astype(np.float32)[:, None]).astype(np.float16)
    pg, sg, zg = cu(packed), cu(scales), cu(zr)
    tiled, tiled_z = hb.w4_repack_tiled(pg, sg, K, 128), hb.w4_repack_tiled(pg, sg, K, 128, zeros=zg)
    q8g, s8g = cu(q8), cu(s8)
    _lib.kernel_status(True)
    for M in (1, 8, 64):
        x = rng.standard_normal((M, K)).astype(np.float16)
        xg = cu(x)
        for name, y, ref in (
                ("w4 tensor-core", hb.w4_tiled_linear(xg, tiled, Nout, K), _dequant_ref(x, W4)),
                ("w4 tensor-core, zero-points", hb.w4_tiled_linear(xg, tiled_z, Nout, K), _dequant_ref(x, W4z)),
                ("w4 gemv", hb.w4_groupwise_linear(xg, pg, sg, Nout, K, group_size=128), _dequant_ref(x, W4)),
                ("w8 gemv", hb.w8_linear(xg, q8g, s8g), _dequant_ref(x, W8))):
            tol = 2e-3 * max(1.0, float(np.abs(ref).max()))
            np.testing.assert_allclose(npf(y).astype(np.float64), ref, rtol=2e-3, atol=tol, err_msg=f"{name} M={M}")
            assert rel_err(npf(y), ref) < 1e-3, (name, M)
    assert _lib.kernel_status(True) == 0


@pytest.mark.parametrize("Nout", [4096, 16384])
def test_config3_int8_gemm_4096_rows_bit_exact(Nout):
    """Prefill GEMM of the A8W8 path at M = 4096, K = 4096: int32 accumulators identical to the exact integer product
    (computed in float64, exact because every partial sum stays below 2^53), and the full a8w8_linear against the
    oracle."""
    M, K = 4096, 4096
    rng = np.random.default_rng(Nout)
    qa = rng.integers(-127, 128, (M, K), dtype=np.int8)
    qw = rng.integers(-127, 128, (Nout, K), dtype=np.int8)
    acc = hb.int8_mm(cu(qa), cu(qw)).cpu().numpy()
    ref = np.rint(qa.astype(np.float64) @ qw.astype(np.float64).T).astype(np.int64)
    assert np.abs(ref).max() < 2 ** 31
    assert np.array_equal(acc.astype(np.int64), ref)
    # a slice of rows through the int64 restatement as well (the two references agree)
    assert np.array_equal(acc[:16], O.int8_gemm_i32(qa[:16], qw.T, exact_int64=True))
    W = (0.02 * rng.standard_normal((Nout, K))).astype(np.float16)
    x = rng.standard_normal((256, K)).astype(np.float16)
    qt, st = O.quantize_weight_per_channel_int8(W)
    yo, acc_o, qa_o, sa_o = O.a8w8_linear(x, qt, st)
    y = hb.a8w8_linear(cu(x), cu(np.ascontiguousarray(qt.T)).t(), cu(st))
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=1e-3, atol=2e-3)


def test_config5_one_layer_at_7p2b_width_against_oracle():
    """Two layers at d_model 4096, 64 heads, FFN 16384 with int4 group-128 projections (one without the v-gate LoRA, one
    with), batch 4, three tokens, fp16: logits cosine >= 0.9995 and state relative error <= 1e-2 against the oracle's
    token step on the same quantised weights."""
    cfg = hb.NativeRWKV7Config(vocab_size=512, hidden_size=4096, num_hidden_layers=2, num_heads=64, head_dim=64,
                               intermediate_size=16384, decay_low_rank_dim=64, a_low_rank_dim=64, v_low_rank_dim=32,
                               gate_low_rank_dim=128)
    model = hb.RWKV7ForCausalLM(cfg)
    sd = seeded_state_dict({k: v.shape for k, v in model.state_dict().items()}, 5, dtype=torch.float16)
    model.load_state_dict(sd)
    model = model.half()
    assert hb.quantize_model(model, "mm4", min_params=1 << 20, group_size=128) == 12
    model = model.cuda().eval()
    g = {"param::" + k: v.numpy() for k, v in sd.items()}
    params = params_from_golden(g)
    for d in params["layers"]:
        for nm in ("Rw", "Kw", "Vw", "Ow", "fK", "fV"):
            p_, s_ = O.quantize_w4_groupwise(d[nm], 128)
            d[nm] = dict(kind="w4g", packed=p_, scales=s_)
    B, H = 4, 64
    ids = np.random.default_rng(3).integers(0, 512, (B, 3))
    cache_o = O.new_cache(2, B, 4096, H, N, np.float16)
    cache = model.new_cache(B)
    for t in range(3):
        lo = O.model_step(params, ids[:, t], cache_o, H, N)
        lg = model.rwkv7_forward_token(cu(ids[:, t]), cache, use_graph=(t == 2))
        a, b = npf(lg).astype(np.float64).ravel(), lo.astype(np.float64).ravel()
        assert a @ b / np.linalg.norm(a) / np.linalg.norm(b) > 0.9995, f"token {t}"
    so = np.stack(cache_o["state"])
    assert np.linalg.norm(npf(torch.stack(cache._state)) - so) / np.linalg.norm(so) < 1e-2
    np.testing.assert_allclose(npf(lg), lo.astype(np.float32), rtol=3e-2, atol=3e-2)


def test_config4_layers_at_2p9b_width_int8_against_oracle():
    """Two layers at d_model 2560, 40 heads, FFN 10240 with per-output-channel int8 on all six projections (the 2.9B
    configuration's format), batch 64 as that configuration decodes it, three tokens, fp16: logits cosine >= 0.9995
    and state relative error <= 1e-2 against the oracle's token step on the same quantised weights; then a 64-token
    prefill chunk of the same model (dequantised weights through the dense GEMM, tensor-core scan) against 64 decode
    steps of it."""
    cfg = hb.NativeRWKV7Config(vocab_size=512, hidden_size=2560, num_hidden_layers=2, num_heads=40, head_dim=64,
                               intermediate_size=10240, decay_low_rank_dim=64, a_low_rank_dim=64, v_low_rank_dim=32,
                               gate_low_rank_dim=128)
    model = hb.RWKV7ForCausalLM(cfg)
    sd = seeded_state_dict({k: v.shape for k, v in model.state_dict().items()}, 6, dtype=torch.float16)
    model.load_state_dict(sd)
    model = model.half()
    assert hb.quantize_model(model, "w8", min_params=1 << 20) == 12
    model = model.cuda().eval()
    g = {"param::" + k: v.numpy() for k, v in sd.items()}
    params = params_from_golden(g)
    for d in params["layers"]:
        for nm in ("Rw", "Kw", "Vw", "Ow", "fK", "fV"):
            q_, s_ = O.quantize_w8_row(d[nm])
            d[nm] = dict(kind="w8", q=q_, s=s_)
    B, H = 64, 40
    ids = np.random.default_rng(4).integers(0, 512, (B, 3))
    cache_o = O.new_cache(2, B, 2560, H, N, np.float16)
    cache = model.new_cache(B)
    for t in range(3):
        lo = O.model_step(params, ids[:, t], cache_o, H, N)
        lg = model.rwkv7_forward_token(cu(ids[:, t]), cache, use_graph=(t == 2))
        a, b = npf(lg).astype(np.float64).ravel(), lo.astype(np.float64).ravel()
        assert a @ b / np.linalg.norm(a) / np.linalg.norm(b) > 0.9995, f"token {t}"
    so = np.stack(cache_o["state"])
    assert np.linalg.norm(npf(torch.stack(cache._state)) - so) / np.linalg.norm(so) < 1e-2
    # prefill chunk == the same tokens one by one (different kernels: GEMM on dequantised weights, chunked scan)
    pids = torch.randint(0, 512, (4, 64), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    lp, cp = model.rwkv7_prefill_native(pids, None, logits_to_keep=1, scan_chunk=64)
    cd = model.new_cache(4)
    for t in range(64):
        ld = model.rwkv7_forward_token(pids[:, t], cd, use_graph=False)
    a, b = npf(lp[:, -1]).astype(np.float64).ravel(), npf(ld).astype(np.float64).ravel()
    assert a @ b / np.linalg.norm(a) / np.linalg.norm(b) > 0.999
    sp, sdec = npf(torch.stack(cp._state)), npf(torch.stack(cd._state))
    assert np.linalg.norm(sp - sdec) / np.linalg.norm(sdec) < 1e-2


def test_a8w8_ffn_against_reference_composition():
    """The fused A8W8 FFN (int8 hidden activation) against the reference's own up -> relu^2 -> down + residual on its
    CPU route (fixture a8w8_ffn.npz), at the reference's gate for this approximation (cosine >= 0.999,
    tests/test_native_quant_a8w8.py:63,92), and against the oracle's restatement of the fused kernels."""
    g = golden("a8w8_ffn.npz")
    D, Fi = g["Wu"].shape[1], g["Wu"].shape[0]
    up_l, down_l = torch.nn.Linear(D, Fi, bias=False), torch.nn.Linear(Fi, D, bias=False)
    with torch.no_grad():
        up_l.weight.copy_(torch.from_numpy(g["Wu"].astype(np.float32)))
        down_l.weight.copy_(torch.from_numpy(g["Wd"].astype(np.float32)))
    up, down = hb.A8W8Linear(up_l.half()).cuda(), hb.A8W8Linear(down_l.half()).cuda()
    assert np.array_equal(up.weight_scale.cpu().numpy(), g["su"]) and np.array_equal(down.weight_scale.cpu().numpy(), g["sd"])
    y = hb.a8w8_ffn(cu(g["x"]), up, down, cu(g["res"]))
    assert y is not None
    a, b = npf(y).astype(np.float64).ravel(), g["y"].astype(np.float64).ravel()
    assert a @ b / np.linalg.norm(a) / np.linalg.norm(b) >= 0.999
    # the residual dominates that cosine: also compare the FFN contribution alone
    fa, fb = a - g["res"].astype(np.float64).ravel(), b - g["res"].astype(np.float64).ravel()
    assert fa @ fb / np.linalg.norm(fa) / np.linalg.norm(fb) >= 0.999
    yo = O.a8w8_ffn(g["x"], up.q_weight_t.cpu().numpy(), g["su"], down.q_weight_t.cpu().numpy(), g["sd"], g["res"])
    yo = yo[0] if isinstance(yo, tuple) else yo
    np.testing.assert_allclose(npf(y), np.asarray(yo, np.float32), rtol=2e-3, atol=4e-3)


@pytest.mark.parametrize("B,T,Hh,chunk", [(2, 16, 2, 16), (3, 48, 2, 16), (2, 80, 3, 16), (2, 96, 1, 32), (2, 144, 2, 16)])
def test_chunk_scan_ragged_tiles(B, T, Hh, chunk):
    """T a multiple of the chunk size but not of the kernel's 64-token tile, more than one sequence: the last tile's
    TMA box reaches into the next sequence's rows (or past the end of the tensor) and the tail must be masked."""
    from hf_adapter_b200 import _lib
    r, w, k, v, kk, a = wkv_inputs(B, T, Hh, N, seed=T * 3 + chunk)
    s0 = (0.1 * np.random.default_rng(T).standard_normal((B, Hh, N, N))).astype(np.float32)
    yo, so = O.recurrent_scan(r, w, k, v, kk, a, s0, hi=True)
    _lib.kernel_status(True)
    y, s = hb.self_chunk_rwkv7(*[cu(t) for t in (r, w, k, v, kk, a, s0)], chunk_size=chunk)
    assert _lib.kernel_status(True) == 0
    assert torch.isfinite(y).all() and torch.isfinite(s).all()
    assert rel_err(npf(s), so) < 1e-3
    assert rel_err(npf(y), yo.astype(np.float32)) < 2e-3


def test_sequence_shift_mix_strict_rounding_and_workspace():
    """strict_fp16_rounding=True == three separately rounded fp16 operations (eager PyTorch on the same device), bit for
    bit; the FFN variant takes its parameters positionally and writes into a [B,T,C] workspace."""
    gen = torch.Generator(device="cuda").manual_seed(4)
    B, T, D = 3, 7, 256
    x = torch.randn(B, T, D, device="cuda", generator=gen).half()
    p0 = torch.randn(B, D, device="cuda", generator=gen).half()
    mixes = [torch.rand(D, device="cuda", generator=gen).half() for _ in range(6)]
    prev = torch.cat([p0[:, None], x[:, :-1]], 1)
    outs = hb.fused_attn_sequence_shift_mix(x, p0, *mixes, strict_fp16_rounding=True)
    for o, m in zip(outs[:6], mixes):
        assert torch.equal(o, x + (prev - x) * m)
    assert torch.equal(outs[6], x[:, -1])
    ws = torch.empty_like(x)
    out, nxt = hb.fused_ffn_sequence_shift_mix(x, p0, mixes[0], 256, 4, ws, True)
    assert out.data_ptr() == ws.data_ptr() and torch.equal(out, x + (prev - x) * mixes[0]) and torch.equal(nxt, x[:, -1])
    loose, _ = hb.fused_ffn_sequence_shift_mix(x, p0, mixes[0])
    np.testing.assert_allclose(npf(loose), npf(out), rtol=2e-3, atol=2e-3)
