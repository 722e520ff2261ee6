"""GPU parity of the operators around the core path: K/V/KK prep, scan with folded state prep, output prep + o_proj,
dense FFN helpers, the affine 8-bit / 4-bit formats and the fused A8W8 FFN boundary, against the reference fixtures
and the oracle."""
import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from oracle import rwkv7_oracle as O
from tests.gpu_util import cu, golden, npf

pytestmark = pytest.mark.gpu
H, N = 2, 64
EPS = N * 1e-5


def _tol(dt):
    return dict(rtol=2e-5, atol=2e-5) if dt == "fp32" else dict(rtol=1e-2, atol=5e-3)


@pytest.mark.parametrize("dt", ["fp32", "fp16"])
def test_composed_operators_against_golden(dt):
    g = golden(f"ops_{dt}.npz")
    tol = _tol(dt)
    k, v, kk = hb.fused_prefill_kv_kk_prep(cu(g["sp_k_raw"]), cu(g["sp_v_raw"]), cu(g["sp_a"]), cu(g["raw_k_k"]),
                                           cu(g["raw_k_a"]), v_first=cu(g["sp_vf"]), v_gate=cu(g["sp_vg"]), num_heads=H,
                                           head_dim=N)
    for mine, ref in ((k, "kvkk_k"), (v, "kvkk_v"), (kk, "kvkk_kk")):
        np.testing.assert_allclose(npf(mine), g[ref].astype(np.float32), **tol)
    # without the v gate (layer 0)
    k0, v0, kk0 = hb.fused_prefill_kv_kk_prep(cu(g["sp_k_raw"]), cu(g["sp_v_raw"]), cu(g["sp_a"]), cu(g["raw_k_k"]),
                                              cu(g["raw_k_a"]), num_heads=H, head_dim=N)
    assert torch.equal(k0, k) and torch.equal(kk0, kk) and torch.equal(v0, cu(g["sp_v_raw"]))
    y, S, k2, v2 = hb.fused_recurrent_scan_state_prep(cu(g["scan_r"]), cu(g["ssp_w_raw"]), cu(g["ssp_k_raw"]),
                                                      cu(g["ssp_v_raw"]), cu(g["ssp_a"]), cu(g["scan_state"]),
                                                      cu(g["raw_k_k"]), cu(g["raw_k_a"]), v_first=cu(g["ssp_vf"]),
                                                      v_gate=cu(g["ssp_vg"]))
    wide = dict(rtol=max(2 * tol["rtol"], 1e-4), atol=max(4 * tol["atol"], 1e-4))
    np.testing.assert_allclose(npf(S), g["ssp_state_out"], **wide)
    np.testing.assert_allclose(npf(y), g["ssp_y"].astype(np.float32), **wide)
    np.testing.assert_allclose(npf(k2), g["ssp_k"].astype(np.float32), **tol)
    np.testing.assert_allclose(npf(v2), g["ssp_v"].astype(np.float32), **tol)
    rows = g["op_rec"].shape[0]
    o = hb.fused_attn_output_project(cu(g["op_rec"]), cu(g["op_r"]).view(rows, H, N), cu(g["op_k"]).view(rows, H, N),
                                     cu(g["op_v"]).view(rows, H, N), cu(g["op_g"]), cu(g["step_r_k"]), cu(g["step_gn_w"]),
                                     cu(g["step_gn_b"]), cu(g["oproj_w"]), cu(g["oproj_b"]), num_heads=H, head_dim=N,
                                     head_v_dim=N, eps=EPS)
    np.testing.assert_allclose(npf(o), g["oproj_out"].astype(np.float32), rtol=max(tol["rtol"], 1e-4), atol=max(tol["atol"], 2e-4))
    mix0 = cu(g["mix_mixes"][0])
    fo, fn = hb.fused_ffn(cu(g["ffn_x"]), cu(g["ffn_prev"]), mix0, cu(g["ffn_key"]), cu(g["ffn_value"]))
    np.testing.assert_allclose(npf(fo), g["ffn_out"].astype(np.float32), rtol=max(tol["rtol"], 1e-4), atol=max(tol["atol"], 1e-4))
    assert np.array_equal(fn.cpu().numpy(), g["ffn_next"])
    so, sn = hb.fused_sequence_ffn(cu(g["sffn_x"]), cu(g["sffn_prev"]), mix0, cu(g["ffn_key"]), cu(g["ffn_value"]))
    np.testing.assert_allclose(npf(so), g["sffn_out"].astype(np.float32), rtol=max(tol["rtol"], 1e-4), atol=max(tol["atol"], 1e-4))
    assert np.array_equal(sn.cpu().numpy(), g["sffn_next"])
    with pytest.raises(ValueError):
        hb.fused_ffn(cu(g["ffn_x"]), cu(g["ffn_prev"]), mix0, cu(g["ffn_value"]), cu(g["ffn_value"]))
    with pytest.raises(RuntimeError):
        hb.fused_ffn(cu(g["ffn_x"]), cu(g["ffn_prev"]), mix0, cu(g["ffn_key"]), cu(g["ffn_value"]), force_fallback=True)


def test_affine_formats_against_golden():
    """Dequantised weights are bit-identical to the reference's (same operation order, every step rounded to fp16);
    the quantisers run on the GPU and give the fixture's bytes."""
    g = golden("quant.npz")
    x = cu(g["x"])
    W8 = hb.dequantize_mm8(cu(g["mm8h_u8"]), cu(g["mm8h_mx"]), cu(g["mm8h_rx"]), cu(g["mm8h_my"]), cu(g["mm8h_ry"]))
    assert np.array_equal(W8.cpu().numpy(), g["mm8h_W"])
    y8 = hb.mm8_matmul(x, cu(g["mm8h_u8"]), cu(g["mm8h_mx"]), cu(g["mm8h_rx"]), cu(g["mm8h_my"]), cu(g["mm8h_ry"]))
    np.testing.assert_allclose(npf(y8), g["mm8h_y"].astype(np.float32), rtol=1e-2, atol=5e-3)
    for tag, m in (("mm4a", 96), ("mm4o", 95)):
        W4 = hb.dequantize_mm4(cu(g[tag + "_packed"]), cu(g[tag + "_mx"]), cu(g[tag + "_rx"]), cu(g[tag + "_my"]),
                               cu(g[tag + "_ry"]), m)
        assert np.array_equal(W4.cpu().numpy(), g[tag + "_W"])
    y4 = hb.mm4_matmul(x, cu(g["mm4a_packed"]), cu(g["mm4a_mx"]), cu(g["mm4a_rx"]), cu(g["mm4a_my"]), cu(g["mm4a_ry"]), 96)
    np.testing.assert_allclose(npf(y4), g["mm4a_y"].astype(np.float32), rtol=1e-2, atol=5e-3)
    Wt = cu(np.ascontiguousarray(g["W"].T))
    u8, mx, rx, my, ry = hb.quantize_mm8(Wt)
    assert np.array_equal(u8.cpu().numpy(), g["mm8h_u8"]) and np.array_equal(rx.cpu().numpy(), g["mm8h_rx"])
    p4, mx4, rx4, my4, ry4, mo, mp = hb.quantize_mm4(Wt[:, :95].contiguous())
    assert (mo, mp) == (95, 96) and np.array_equal(p4.cpu().numpy(), g["mm4o_packed"])
    assert np.array_equal(ry4.cpu().numpy(), g["mm4o_ry"])


@pytest.mark.parametrize("M", [1, 3, 8, 20, 40])
@pytest.mark.parametrize("K,Nn", [(256, 96), (1024, 264), (4096, 4096)])
def test_affine_gemv_against_oracle(M, K, Nn):
    """The weight-streaming kernel (1..32 rows) and the dequantise-then-GEMM route (more rows), both bit widths."""
    rng = np.random.default_rng(M * 131 + K + Nn)
    W = (0.02 * rng.standard_normal((K, Nn))).astype(np.float16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    u8, mx, rx, my, ry = O.quantize_mm8(W.astype(np.float32))
    f16 = lambda a: np.asarray(a, np.float16)
    mx, rx, my, ry = f16(mx), f16(rx), f16(my), f16(ry)
    yo = O.mm8_matmul(x, u8, mx, rx, my, ry, hi=True).astype(np.float32)
    y = hb.mm8_matmul(cu(x), cu(u8), cu(mx), cu(rx), cu(my), cu(ry))
    tol = 4e-3 * max(1.0, float(np.abs(yo).max()))
    np.testing.assert_allclose(npf(y), yo, rtol=4e-3, atol=tol)
    assert torch.equal(hb.mm8_matmul(cu(x), cu(u8), cu(mx), cu(rx), cu(my), cu(ry)), y)  # deterministic
    p4, mx4, rx4, my4, ry4, m, mp = O.quantize_mm4(W)
    y4o = O.mm4_matmul(x, p4, mx4, rx4, my4, ry4, m, hi=True).astype(np.float32)
    y4 = hb.mm4_matmul(cu(x), cu(p4), cu(mx4), cu(rx4), cu(my4), cu(ry4), m)
    np.testing.assert_allclose(npf(y4), y4o, rtol=4e-3, atol=4e-3 * max(1.0, float(np.abs(y4o).max())))
    # the module: reference buffer names, same result, epilogue hooks
    lin = torch.nn.Linear(K, Nn, bias=False)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(W.T.astype(np.float32)))
    mod = hb.MM8Linear(lin.half()).cuda()
    assert np.array_equal(mod.w_u8.cpu().numpy(), u8)
    assert torch.equal(mod(cu(x)), y)
    res = cu(rng.standard_normal((M, Nn)).astype(np.float16))
    np.testing.assert_allclose(npf(mod.rwkv7_forward_add(cu(x), res)), yo + npf(res), rtol=4e-3, atol=2 * tol)
    r2 = (np.maximum(yo.astype(np.float16).astype(np.float32), 0) ** 2)
    np.testing.assert_allclose(npf(mod.rwkv7_forward_relu2(cu(x))), r2, rtol=1e-2, atol=8e-3 * max(1.0, float(r2.max())))


@pytest.mark.parametrize("M", [1, 17, 64, 200])
def test_a8w8_fused_ffn_against_oracle(M):
    """up GEMM -> (dequantise, fp16 relu^2, requantise) -> down GEMM + residual: the boundary kernel is bit-exact
    against the oracle, the whole chain follows it."""
    rng = np.random.default_rng(M)
    D, Fi = 256, 1024
    Wu = (0.05 * rng.standard_normal((Fi, D))).astype(np.float16)
    Wd = (0.05 * rng.standard_normal((D, Fi))).astype(np.float16)
    x = rng.standard_normal((M, D)).astype(np.float16)
    res = rng.standard_normal((M, D)).astype(np.float16)
    qu, su = O.quantize_weight_per_channel_int8(Wu)
    qd, sd = O.quantize_weight_per_channel_int8(Wd)
    yo, qh_o, sh_o = O.a8w8_ffn(x, qu, su, qd, sd, res)
    mk = lambda W: torch.nn.Linear(W.shape[1], W.shape[0], bias=False)
    up, down = mk(Wu), mk(Wd)
    with torch.no_grad():
        up.weight.copy_(torch.from_numpy(Wu.astype(np.float32)))
        down.weight.copy_(torch.from_numpy(Wd.astype(np.float32)))
    up, down = hb.A8W8Linear(up.half()).cuda(), hb.A8W8Linear(down.half()).cuda()
    # the boundary kernel alone
    from hf_adapter_b200 import _lib
    from hf_adapter_b200._util import ptr, stream_ptr
    qa, sa = hb.dynamic_a8_quant(cu(x))
    acc = hb.int8_mm(qa, up.q_weight_t.t())
    qh = torch.empty((M, Fi), device="cuda", dtype=torch.int8)
    sh = torch.empty((M,), device="cuda", dtype=torch.float32)
    _lib.check(_lib.lib.rwkv7_a8w8_relu2_requant(ptr(acc), ptr(sa), ptr(up.weight_scale), None, ptr(qh), ptr(sh), M, Fi, 0,
                                                 stream_ptr(acc)), "relu2_requant")
    assert np.array_equal(sh.cpu().numpy(), sh_o) and np.array_equal(qh.cpu().numpy(), qh_o)
    y = hb.a8w8_ffn(cu(x), up, down, cu(res))
    assert y is not None
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=2e-3, atol=2e-3)
    assert torch.equal(up.rwkv7_forward_ffn(cu(x), down, cu(res)), y)
    # contract violations fall back to None like the reference
    assert hb.a8w8_ffn(cu(x).float(), up, down, cu(res)) is None
    assert hb.a8w8_ffn(cu(x), up, torch.nn.Linear(Fi, D).cuda().half(), cu(res)) is None


@pytest.mark.parametrize("shape", [(3, 128), (2, 5, 256)])
def test_attn_shift_mix_explicit_previous(shape):
    """out_i = x + (prev - x) * mix_i for the six streams, any leading shape, mix vectors of any shape with D elements."""
    rng = np.random.default_rng(sum(shape))
    x, prev = (rng.standard_normal(shape).astype(np.float16) for _ in range(2))
    mixes = [rng.random((1, 1, shape[-1])).astype(np.float16) for _ in range(6)]
    outs = hb.fused_attn_shift_mix(cu(x), cu(prev), *(cu(m) for m in mixes))
    assert len(outs) == 6
    for o, m in zip(outs, mixes):
        ref = x.astype(np.float32) + (prev.astype(np.float32) - x.astype(np.float32)) * m.reshape(-1).astype(np.float32)
        assert tuple(o.shape) == shape
        np.testing.assert_allclose(npf(o), ref, rtol=2e-3, atol=2e-3)
    with pytest.raises(ValueError):
        hb.fused_attn_shift_mix(cu(x), cu(prev)[:1], *(cu(m) for m in mixes))
