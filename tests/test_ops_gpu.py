"""GPU parity of the recurrence / norm-mix / LoRA / prep kernels, called through the C ABI via the
reference-signature wrappers, against (a) the golden outputs of the reference and (b) the pinned oracle on
fresh seeded inputs, including ragged and edge shapes."""
import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from oracle import rwkv7_oracle as O
from tests.gpu_util import cu, golden, npf, rel_err, wkv_inputs

pytestmark = pytest.mark.gpu
H, N = 2, 64
EPS = N * 1e-5
TD = {"fp32": torch.float32, "fp16": torch.float16}


def tol(dt, k=1.0):
    return dict(rtol=3e-5 * k, atol=3e-5 * k) if dt == "fp32" else dict(rtol=4e-3 * k, atol=4e-3 * k)


@pytest.mark.parametrize("dt", ["fp32", "fp16"])
def test_step_against_golden(dt):
    g = golden(f"ops_{dt}.npz")
    t = {k: cu(v) for k, v in g.items() if k.startswith(("step_", "raw_"))}
    y, s = hb.fused_recurrent_update(t["step_r"], t["step_w"], t["step_k"], t["step_v"], t["step_kk"], t["step_a"], t["step_state"])
    st = dict(rtol=1e-4, atol=1e-4) if dt == "fp32" else dict(rtol=1e-2, atol=5e-3)
    np.testing.assert_allclose(npf(s), g["step_state_out"], **st)
    np.testing.assert_allclose(npf(y), g["step_y"].astype(np.float32), **tol(dt, 20))
    assert y.dtype == TD[dt] and s.dtype == torch.float32 and tuple(y.shape) == (2, H, N)
    # flat inputs -> flat output; the input state must be untouched
    s_before = t["step_state"].clone()
    y2, s2 = hb.fused_recurrent_update(*(t[f"step_{n}"].reshape(2, H * N) for n in ("r", "w", "k", "v", "kk", "a")), t["step_state"])
    assert tuple(y2.shape) == (2, H * N) and torch.equal(y2.reshape(2, H, N), y) and torch.equal(s2, s)
    assert torch.equal(t["step_state"], s_before)
    yp, sp = hb.fused_recurrent_output_prepare(t["step_r"], t["step_w"], t["step_k"], t["step_v"], t["step_kk"], t["step_a"],
                                               t["step_state"], t["step_g"], t["step_r_k"], t["step_gn_w"], t["step_gn_b"], eps=EPS)
    np.testing.assert_allclose(npf(yp), g["prep_y"].astype(np.float32), **tol(dt, 3))
    yr, sr = hb.fused_recurrent_output_prepare_raw(t["step_r"], t["raw_w"], t["raw_k"], t["step_v"], t["step_a"], t["step_state"],
                                                   t["step_g"], t["raw_k_k"], t["raw_k_a"], t["step_r_k"], t["step_gn_w"],
                                                   t["step_gn_b"], eps=EPS)
    np.testing.assert_allclose(npf(yr), g["raw_y"].astype(np.float32), **tol(dt, 3))
    np.testing.assert_allclose(npf(sr), g["raw_state_out"], **st)


@pytest.mark.parametrize("B,Hh", [(1, 1), (3, 5), (64, 8)])
def test_step_against_oracle_and_inplace(B, Hh):
    r, w, k, v, kk, a = (x[:, 0] for x in wkv_inputs(B, 1, Hh, N, seed=B * 31 + Hh))
    rng = np.random.default_rng(5)
    state = (0.3 * rng.standard_normal((B, Hh, N, N))).astype(np.float32)
    g = rng.standard_normal((B, Hh, N)).astype(np.float16)
    w_raw = rng.standard_normal((B, Hh, N)).astype(np.float16)
    k_k = (0.85 + 0.1 * rng.standard_normal(Hh * N)).astype(np.float16)
    k_a = (1 + 0.1 * rng.standard_normal(Hh * N)).astype(np.float16)
    r_k = (0.1 * rng.standard_normal((Hh, N))).astype(np.float16)
    gw = (1 + 0.1 * rng.standard_normal(Hh * N)).astype(np.float16)
    gb = (0.1 * rng.standard_normal(Hh * N)).astype(np.float16)
    yo, so = O.recurrent_output_prepare_raw(r, w_raw, k, v, a, state, g, k_k, k_a, r_k, gw, gb, EPS)
    args = [cu(x) for x in (r, w_raw, k, v, a)]
    st = cu(state)
    par = [cu(x) for x in (g, k_k, k_a, r_k, gw, gb)]
    y, s = hb.fused_recurrent_output_prepare_raw(*args, st, *par, eps=EPS)
    np.testing.assert_allclose(npf(s), so, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=4e-3, atol=4e-3)
    # in-place variant gives bit-identical results
    st2 = st.clone()
    y2, s2 = hb.fused_recurrent_output_prepare_raw(*args, st2, *par, eps=EPS, new_state=st2)
    assert s2.data_ptr() == st2.data_ptr() and torch.equal(st2, s) and torch.equal(y2, y)
    # repeatability (no atomics, fixed reduction order)
    y3, s3 = hb.fused_recurrent_output_prepare_raw(*args, st, *par, eps=EPS)
    assert torch.equal(y3, y) and torch.equal(s3, s)


def test_back_to_back_steps_feed_each_other():
    """Twelve one-token updates launched back to back, each reading the state the previous launch wrote in place
    (the kernels are launched programmatically: a launch must wait for its predecessor before it loads the state),
    against the oracle's sequential scan."""
    B, T, Hh = 64, 12, 32
    r, w, k, v, kk, a = wkv_inputs(B, T, Hh, N, seed=77)
    state = (0.3 * np.random.default_rng(6).standard_normal((B, Hh, N, N))).astype(np.float32)
    yo, so = O.recurrent_scan(r, w, k, v, kk, a, state)
    dev = [cu(x) for x in (r, w, k, v, kk, a)]
    st = cu(state)
    steps = [[x[:, t].contiguous() for x in dev] for t in range(T)]  # sliced first: no other kernel between the launches
    outs = [hb.fused_recurrent_update(*steps[t], st, new_state=st)[0] for t in range(T)]
    np.testing.assert_allclose(npf(st), so, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(npf(torch.stack(outs, 1)), yo.astype(np.float32), rtol=4e-3, atol=4e-3)


def test_step_fused_lora_epilogues():
    """w/a biases, sigmoids and the v_first interpolation folded into the step == doing them beforehand."""
    B, Hh = 4, 3
    rng = np.random.default_rng(11)
    f16 = lambda *s: rng.standard_normal(s).astype(np.float16)
    r, w_pre, k, v, a_pre, g, vg_pre, vf = (f16(B, Hh, N) for _ in range(8))
    wb, ab, vb = (0.5 * f16(Hh * N) for _ in range(3))
    k_k, k_a, r_k, gw, gb = (0.85 + 0.1 * f16(Hh * N)), (1 + 0.1 * f16(Hh * N)), 0.1 * f16(Hh, N), 1 + 0.1 * f16(Hh * N), 0.1 * f16(Hh * N)
    state = (0.3 * rng.standard_normal((B, Hh, N, N))).astype(np.float32)
    h = lambda x: np.asarray(x, np.float16)
    w_raw = h(w_pre.astype(np.float32) + wb.reshape(Hh, N).astype(np.float32))
    a = h(O.sigmoid(h(a_pre.astype(np.float32) + ab.reshape(Hh, N).astype(np.float32)).astype(np.float32)))
    gate = h(O.sigmoid(h(vg_pre.astype(np.float32) + vb.reshape(Hh, N).astype(np.float32)).astype(np.float32)))
    v_mix = h(v.astype(np.float32) + (vf.astype(np.float32) - v.astype(np.float32)) * gate.astype(np.float32))
    yo, so = O.recurrent_output_prepare_raw(r, w_raw, k, v_mix, a, state, g, h(k_k), h(k_a), h(r_k), h(gw), h(gb), EPS)
    v_out = torch.empty((B, Hh * N), device="cuda", dtype=torch.float16)
    y, s = hb.fused_recurrent_output_prepare_raw(
        cu(r), cu(w_pre), cu(k), cu(v), cu(a_pre), cu(state), cu(g), cu(h(k_k)), cu(h(k_a)), cu(h(r_k)), cu(h(gw)), cu(h(gb)),
        eps=EPS, w_bias=cu(h(wb)), a_bias=cu(h(ab)), a_is_raw=True, v_first=cu(vf), v_gate=cu(vg_pre),
        v_gate_bias=cu(h(vb)), v_gate_is_raw=True, v_out=v_out)
    np.testing.assert_allclose(npf(v_out).reshape(B, Hh, N), v_mix.astype(np.float32), rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(npf(s), so, rtol=1e-2, atol=3e-3)
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dt", ["fp32", "fp16"])
def test_scan_against_golden(dt):
    g = golden(f"ops_{dt}.npz")
    a = [cu(g[f"scan_{n}"]) for n in ("r", "w", "k", "v", "kk", "a", "state")]
    y, s = hb.fused_recurrent_scan(*a)
    np.testing.assert_allclose(npf(s), g["scan_state_out"], rtol=1e-4, atol=1e-4 if dt == "fp32" else 5e-3)
    np.testing.assert_allclose(npf(y), g["scan_y"].astype(np.float32), rtol=1e-4 if dt == "fp32" else 1e-2, atol=2e-4 if dt == "fp32" else 3e-2)
    yp, sp = hb.fused_recurrent_scan_output_prepare(*a, cu(g["scan_g"]), cu(g["step_r_k"]), cu(g["step_gn_w"]), cu(g["step_gn_b"]), eps=EPS)
    np.testing.assert_allclose(npf(yp), g["scanprep_y"].astype(np.float32), rtol=1e-3 if dt == "fp32" else 2e-2, atol=1e-3 if dt == "fp32" else 3e-2)
    assert torch.equal(sp, s)


@pytest.mark.parametrize("B,T,Hh", [(1, 1, 1), (2, 17, 3), (3, 33, 2), (2, 130, 4)])
def test_scan_against_oracle_ragged(B, T, Hh):
    r, w, k, v, kk, a = wkv_inputs(B, T, Hh, N, seed=T)
    rng = np.random.default_rng(T + 1)
    s0 = (0.1 * rng.standard_normal((B, Hh, N, N))).astype(np.float32)
    yo, so = O.recurrent_scan(r, w, k, v, kk, a, s0)
    y, s = hb.fused_recurrent_scan(*(cu(x) for x in (r, w, k, v, kk, a, s0)))
    assert rel_err(npf(s), so) < 2e-5
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=4e-3, atol=4e-3)
    # T single-step calls == scan (config-2 protocol), final state relative error <= 1e-3
    st = cu(s0)
    ys = []
    for t in range(T):
        yt, st = hb.fused_recurrent_update(*(cu(x[:, t]) for x in (r, w, k, v, kk, a)), st)
        ys.append(yt)
    assert rel_err(npf(st), so) < 1e-3
    np.testing.assert_allclose(npf(torch.stack(ys, 1)), npf(y), rtol=4e-3, atol=4e-3)
    # decay given in the activation dtype, and raw-w (clampw) variant
    y16, s16 = hb.fused_recurrent_scan(cu(r), cu(w.astype(np.float16)), *(cu(x) for x in (k, v, kk, a, s0)))
    yo16, so16 = O.recurrent_scan(r, w.astype(np.float16), k, v, kk, a, s0)
    assert rel_err(npf(s16), so16) < 2e-5
    w_raw = rng.standard_normal((B, T, Hh, N)).astype(np.float16)
    yc, sc = hb.fused_recurrent_scan_clampw(cu(r), cu(w_raw), *(cu(x) for x in (k, v, kk, a, s0)))
    wd = np.exp(-0.606531 * O.sigmoid(w_raw.astype(np.float32)))
    yoc, soc = O.recurrent_scan(r, wd, k, v, kk, a, s0)
    assert rel_err(npf(sc), soc) < 2e-5


def test_scan_empty_sequence_passes_state_through():
    s0 = torch.randn(2, 2, N, N, device="cuda")
    e = torch.empty(2, 0, 2, N, device="cuda", dtype=torch.float16)
    y, s = hb.fused_recurrent_scan(e, e.float(), e, e, e, e, s0)
    assert tuple(y.shape) == (2, 0, 2, N) and torch.equal(s, s0)


@pytest.mark.parametrize("dt", ["fp32", "fp16"])
def test_norm_mix_lora_prep_against_golden(dt):
    g = golden(f"ops_{dt}.npz")
    t = {k: cu(v) for k, v in g.items()}
    prev = t["mix_prev"].clone()
    outs = hb.fused_attn_norm_mix6_decode(t["mix_x"], prev, t["mix_nw"], t["mix_nb"], *t["mix_mixes"])
    np.testing.assert_allclose(npf(torch.stack(outs)), g["mix_outs"].astype(np.float32), **tol(dt))
    np.testing.assert_allclose(npf(prev), g["mix_prev_out"].astype(np.float32), **tol(dt))
    for kw in ({"stack_rkv": True}, {"stack_wav": True}, {"stack_rkv_wagv": True}):
        prev2 = t["mix_prev"].clone()
        outs2 = hb.fused_attn_norm_mix6_decode(t["mix_x"], prev2, t["mix_nw"], t["mix_nb"], *t["mix_mixes"], **kw)
        assert all(torch.equal(a, b) for a, b in zip(outs, outs2))
    prev = t["mix_prev"].clone()
    x, mixed = hb.fused_ffn_add_norm_mix_decode(t["mix_x"], t["ffnmix_attn"], prev, t["mix_nw"], t["mix_nb"], t["mix_mixes"][0])
    np.testing.assert_allclose(npf(x), g["ffnmix_res_out"].astype(np.float32), **tol(dt))
    np.testing.assert_allclose(npf(mixed), g["ffnmix_mixed"].astype(np.float32), **tol(dt, 3))
    np.testing.assert_allclose(npf(prev), g["ffnmix_prev_out"].astype(np.float32), **tol(dt, 3))
    seq = hb.fused_attn_sequence_shift_mix(t["seqmix_x"], t["seqmix_prev"], *t["mix_mixes"])
    np.testing.assert_allclose(npf(torch.stack(seq[:6])), g["seqmix_outs"].astype(np.float32), **tol(dt))
    assert torch.equal(seq[6], t["seqmix_next"])
    one, nxt = hb.fused_ffn_sequence_shift_mix(t["seqmix_x"], t["seqmix_prev"], t["mix_mixes"][2])
    assert torch.equal(one, seq[2]) and torch.equal(nxt, seq[6])
    w, a, gg, vg = hb.fused_wavg_lora(t["lora_xw"], t["lora_xa"], t["lora_xg"], t["lora_xv"], t["lora_wd"], t["lora_ad"],
                                      t["lora_gd"], t["lora_vd"], t["lora_wu"], t["lora_au"], t["lora_gu"], t["lora_vu"],
                                      t["lora_wb"], t["lora_ab"], None, t["lora_vb"])
    for mine, ref in ((w, "lora_w"), (a, "lora_a"), (gg, "lora_g"), (vg, "lora_vgate")):
        np.testing.assert_allclose(npf(mine), g[ref].astype(np.float32), **tol(dt, 2))
    pw, pk, pv, pkk = hb.fused_prefill_state_prep(t["sp_w_raw"], t["sp_k_raw"], t["sp_v_raw"], t["sp_a"], t["raw_k_k"], t["raw_k_a"],
                                                  v_first=t["sp_vf"], v_gate=t["sp_vg"], num_heads=H, head_dim=N)
    np.testing.assert_allclose(npf(pw), g["sp_w"], rtol=1e-5, atol=1e-6)
    for mine, ref in ((pk, "sp_k"), (pv, "sp_v"), (pkk, "sp_kk")):
        np.testing.assert_allclose(npf(mine), g[ref].astype(np.float32), **tol(dt))
    op = hb.fused_attn_output_prepare(t["op_rec"], t["op_r"], t["op_k"], t["op_v"], t["op_g"], t["step_r_k"], t["step_gn_w"],
                                      t["step_gn_b"], num_heads=H, head_dim=N, head_v_dim=N, eps=EPS)
    np.testing.assert_allclose(npf(op), g["op_out"].astype(np.float32), **tol(dt, 5))


@pytest.mark.parametrize("rows,D", [(1, 8), (5, 768), (64, 4096), (3, 8192)])
def test_norm_mix_shapes(rows, D):
    rng = np.random.default_rng(D)
    f = lambda *s: rng.standard_normal(s).astype(np.float16)
    x, prev, attn = f(rows, D), f(rows, D), f(rows, D)
    nw, nb = (1 + 0.1 * f(D)).astype(np.float16), (0.1 * f(D)).astype(np.float16)
    mixes = [rng.random(D).astype(np.float16) for _ in range(6)]
    (outs_o, prev_o) = O.attn_norm_mix6_decode(x, prev, nw, nb, mixes)
    pv = cu(prev)
    outs = hb.fused_attn_norm_mix6_decode(cu(x), pv, cu(nw), cu(nb), *(cu(m) for m in mixes))
    np.testing.assert_allclose(npf(torch.stack(outs)), np.stack(outs_o).astype(np.float32), rtol=4e-3, atol=4e-3)
    np.testing.assert_allclose(npf(pv), prev_o.astype(np.float32), rtol=4e-3, atol=4e-3)
    xo, mo, po = O.ffn_add_norm_mix_decode(x, attn, prev, nw, nb, mixes[0])
    pv = cu(prev)
    xg, mg = hb.fused_ffn_add_norm_mix_decode(cu(x), cu(attn), pv, cu(nw), cu(nb), cu(mixes[0]))
    np.testing.assert_allclose(npf(xg), xo.astype(np.float32), rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(npf(mg), mo.astype(np.float32), rtol=4e-3, atol=6e-3)
    ln = hb.layer_norm(cu(x), cu(nw), cu(nb))
    np.testing.assert_allclose(npf(ln), O.layer_norm(x, nw, nb).astype(np.float32), rtol=4e-3, atol=4e-3)


@pytest.mark.parametrize("M", [1, 5, 64, 130])
def test_grouped_lora_gemm_against_oracle(M):
    """The one-launch grouped projection (tensor-core MMA, cluster split-K) for decode-size LoRA shapes."""
    from hf_adapter_b200.lora import small_gemm_group
    rng = np.random.default_rng(M)
    D, A = 4096, 512
    ranks = (64, 64, 128, 32)
    f = lambda *s, sc=1.0: (sc * rng.standard_normal(s)).astype(np.float16)
    xs = [f(M, D) for _ in ranks]
    downs = [f(r, D, sc=0.02) for r in ranks]
    ups = [f(A, r, sc=0.1) for r in ranks]
    biases = [f(A, sc=0.5), f(A, sc=0.5), None, f(A, sc=0.5)]
    wo, ao, go, vo = O.wavg_lora(xs[0], xs[1], xs[2], xs[3], downs, ups, biases)
    w, a, g, v = hb.fused_wavg_lora(*(cu(x) for x in xs), *(cu(d) for d in downs), *(cu(u) for u in ups),
                                    *(None if b is None else cu(b) for b in biases))
    for mine, ref in ((w, wo), (a, ao), (g, go), (v, vo)):
        np.testing.assert_allclose(npf(mine), ref.astype(np.float32), rtol=4e-3, atol=4e-3)
    again = hb.fused_wavg_lora(*(cu(x) for x in xs), *(cu(d) for d in downs), *(cu(u) for u in ups),
                               *(None if b is None else cu(b) for b in biases))
    assert all(torch.equal(p, q) for p, q in zip((w, a, g, v), again))
    # odd output width / K not a multiple of the 64-wide chunk
    x1, w1, b1 = f(M, 72), f(40, 72, sc=0.1), f(40)
    (y1,) = small_gemm_group((cu(x1),), (cu(w1),), (cu(b1),), acts=(1,))
    ref = np.tanh((x1.astype(np.float32) @ w1.astype(np.float32).T + b1.astype(np.float32)).astype(np.float16).astype(np.float32))
    np.testing.assert_allclose(npf(y1), ref, rtol=4e-3, atol=4e-3)


@pytest.mark.parametrize("B,T,Hh,chunk", [(1, 64, 1, 64), (2, 128, 3, 16), (2, 192, 2, 32), (1, 1024, 2, 64)])
def test_chunk_scan_tensor_core_against_oracle(B, T, Hh, chunk):
    """tcgen05 chunked WY scan == the sequential recurrence (fp64 oracle on the same fp16 inputs):
    state relative error <= 1e-3, outputs within fp16 tolerance, no bounded wait gave up."""
    from hf_adapter_b200 import _lib
    r, w, k, v, kk, a = wkv_inputs(B, T, Hh, N, seed=T + chunk)
    rng = np.random.default_rng(T)
    s0 = (0.1 * rng.standard_normal((B, Hh, N, N))).astype(np.float32)
    yo, so = O.recurrent_scan(r, w, k, v, kk, a, s0, hi=True)
    _lib.kernel_status(True)
    args = [cu(x) for x in (r, w, k, v, kk, a, s0)]
    y, s = hb.self_chunk_rwkv7(*args, chunk_size=chunk)
    assert _lib.kernel_status(True) == 0
    assert rel_err(npf(s), so) < 1e-3
    scale = max(1.0, float(np.abs(yo.astype(np.float32)).max()))
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=4e-3, atol=4e-3 * scale)
    assert rel_err(npf(y), yo.astype(np.float32)) < 2e-3
    y2, s2 = hb.dplr_chunk_scan(*args, chunk_size=chunk, algorithm="wy")
    assert torch.equal(y2, y) and torch.equal(s2, s)
    # the sequential kernel and the chunked kernel agree with each other as well
    y3, s3 = hb.fused_recurrent_scan(*args)
    assert rel_err(npf(s3), npf(s)) < 1e-3
    # decay in the activation dtype / raw w
    y16, s16 = hb.self_chunk_rwkv7(args[0], cu(w.astype(np.float16)), *args[2:], chunk_size=chunk)
    yo16, so16 = O.recurrent_scan(r, w.astype(np.float16), k, v, kk, a, s0, hi=True)
    assert rel_err(npf(s16), so16) < 1e-3
    with pytest.raises(ValueError):
        hb.self_chunk_rwkv7(*args, chunk_size=48)


def test_scan_full_size_config2():
    """Isolated WKV-7 op at the benchmark's size (B8 T4096 H32 N64, zero state): chunked tensor-core scan vs the
    sequential kernel over all heads (state rel-err <= 1e-3, outputs <= 2e-3 relative), and both against the fp64
    oracle on a two-head slice (the oracle needs seconds per head at this length)."""
    B, T, Hh = 8, 4096, 32
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    r, k, v = (rn(B, T, Hh, N).half() for _ in range(3))
    kk = torch.nn.functional.normalize(k.float(), dim=-1).half()
    a = torch.sigmoid(rn(B, T, Hh, N)).half()
    w = torch.exp(-0.606531 * torch.sigmoid(rn(B, T, Hh, N)))
    s0 = torch.zeros(B, Hh, N, N, device="cuda")
    ys, ss = hb.fused_recurrent_scan(r, w, k, v, kk, a, s0)
    yc, sc = hb.self_chunk_rwkv7(r, w, k, v, kk, a, s0, chunk_size=64)
    assert rel_err(npf(sc), npf(ss)) < 1e-3
    assert rel_err(npf(yc), npf(ys)) < 2e-3
    sl = lambda t: t[:1, :, :2].contiguous().cpu().numpy()
    yo, so = O.recurrent_scan(sl(r), sl(w), sl(k), sl(v), sl(kk), sl(a), np.zeros((1, 2, N, N), np.float32), hi=True)
    for s_gpu, y_gpu in ((ss, ys), (sc, yc)):
        assert rel_err(npf(s_gpu[:1, :2]), so) < 1e-3
        assert rel_err(npf(y_gpu[:1, :, :2]), yo.astype(np.float32)) < 2e-3


def test_bf16_activations():
    """The CUDA-core kernels and the LoRA MMA kernel take bf16 storage as well (fp32 arithmetic inside)."""
    rng = np.random.default_rng(21)
    B, Hh, D = 3, 2, 256
    bf = lambda a: torch.from_numpy(np.asarray(a, np.float32)).cuda().to(torch.bfloat16)
    rt = lambda t: t.float().cpu().numpy()  # bf16-rounded values as fp32 for the oracle
    r, w_raw, k, v, g = (bf(rng.standard_normal((B, Hh, N))) for _ in range(5))
    a = bf(1 / (1 + np.exp(-rng.standard_normal((B, Hh, N)))))
    state = (0.3 * rng.standard_normal((B, Hh, N, N))).astype(np.float32)
    k_k, k_a = bf(0.85 + 0.1 * rng.standard_normal(Hh * N)), bf(1 + 0.1 * rng.standard_normal(Hh * N))
    r_k, gw, gb = bf(0.1 * rng.standard_normal((Hh, N))), bf(1 + 0.1 * rng.standard_normal(Hh * N)), bf(0.1 * rng.standard_normal(Hh * N))
    yo, so = O.recurrent_output_prepare_raw(rt(r), rt(w_raw), rt(k), rt(v), rt(a), state, rt(g), rt(k_k), rt(k_a), rt(r_k), rt(gw), rt(gb), EPS)
    y, s = hb.fused_recurrent_output_prepare_raw(r, w_raw, k, v, a, cu(state), g, k_k, k_a, r_k, gw, gb, eps=EPS)
    assert y.dtype == torch.bfloat16
    np.testing.assert_allclose(npf(s), so, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(npf(y), yo, rtol=2e-2, atol=2e-2)
    x, prev = bf(rng.standard_normal((B, D))), bf(rng.standard_normal((B, D)))
    nw, nb = bf(1 + 0.1 * rng.standard_normal(D)), bf(0.1 * rng.standard_normal(D))
    mixes = [bf(rng.random(D)) for _ in range(6)]
    outs_o, prev_o = O.attn_norm_mix6_decode(rt(x), rt(prev), rt(nw), rt(nb), [rt(m) for m in mixes])
    pv = prev.clone()
    outs = hb.fused_attn_norm_mix6_decode(x, pv, nw, nb, *mixes)
    np.testing.assert_allclose(npf(torch.stack(outs)), np.stack(outs_o), rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(npf(pv), prev_o, rtol=2e-2, atol=2e-2)
    from hf_adapter_b200.lora import small_gemm_group
    W = bf(0.05 * rng.standard_normal((72, D)))
    (yl,) = small_gemm_group((x,), (W,), acts=(2,))
    ref = 1 / (1 + np.exp(-(rt(x) @ rt(W).T)))
    np.testing.assert_allclose(npf(yl), ref, rtol=2e-2, atol=2e-2)
    # scan in bf16 storage
    T = 20
    rs, ks, vs = (bf(rng.standard_normal((B, T, Hh, N))) for _ in range(3))
    kks = bf(rt(ks) / np.linalg.norm(rt(ks), axis=-1, keepdims=True))
    as_ = bf(1 / (1 + np.exp(-rng.standard_normal((B, T, Hh, N)))))
    ws = np.exp(-0.606531 / (1 + np.exp(-rng.standard_normal((B, T, Hh, N))))).astype(np.float32)
    yo2, so2 = O.recurrent_scan(rt(rs), ws, rt(ks), rt(vs), rt(kks), rt(as_), state)
    y2, s2 = hb.fused_recurrent_scan(rs, cu(ws), ks, vs, kks, as_, cu(state))
    assert rel_err(npf(s2), so2) < 2e-5
    np.testing.assert_allclose(npf(y2), yo2, rtol=2e-2, atol=3e-2)
