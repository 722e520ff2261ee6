"""GPU parity of the FP16-state lane: the output-prepare operators and the scans with a float16 recurrent state, and the
two entry points of the reference's native_wkv_fp16 extension (decay dither phased by ``elapsed``), against the oracle's
restatement of the reference kernels and against the fp32-state operators at the reference's own gates for this lane
(tests/test_fused_recurrent_output_raw.py:44-141: state atol 3e-3 / rtol 1e-2, output cosine >= 0.999)."""
import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from oracle import rwkv7_oracle as O
from tests.gpu_util import cu, npf, rel_err, wkv_inputs

pytestmark = pytest.mark.gpu
N = 64
EPS = N * 1e-5
h = lambda x: np.asarray(x, np.float16)


def _case(B, Hh, seed):
    rng = np.random.default_rng(seed)
    r, w_raw, k_raw, v, g = (h(0.2 * rng.standard_normal((B, Hh, N))) for _ in range(5))
    a = h(1 / (1 + np.exp(-rng.standard_normal((B, Hh, N)))))
    s32 = (0.1 * rng.standard_normal((B, Hh, N, N))).astype(np.float32)
    k_k, k_a, r_k = h(rng.standard_normal((Hh, N))), h(0.1 * rng.standard_normal((Hh, N))), h(0.1 * rng.standard_normal((Hh, N)))
    nw, nb = h(rng.standard_normal(Hh * N)), h(rng.standard_normal(Hh * N))
    return r, w_raw, k_raw, v, a, s32, g, k_k, k_a, r_k, nw, nb


def _cos_min(a, b):
    a, b = np.asarray(a, np.float64).reshape(a.shape[0], -1), np.asarray(b, np.float64).reshape(b.shape[0], -1)
    return float(((a * b).sum(1) / np.linalg.norm(a, axis=1) / np.linalg.norm(b, axis=1)).min())


@pytest.mark.parametrize("B,Hh", [(2, 3), (64, 8)])
def test_output_prepare_raw_with_fp16_state(B, Hh):
    r, w_raw, k_raw, v, a, s32, g, k_k, k_a, r_k, nw, nb = _case(B, Hh, B + Hh)
    s16 = s32.astype(np.float16)
    dev = [cu(x) for x in (r, w_raw, k_raw, v, a)]
    par = [cu(x) for x in (g, k_k.reshape(-1), k_a.reshape(-1), r_k, nw, nb)]
    # (1) no dither: fp32 arithmetic on the fp16 state == the oracle's fp32 operator run on the same fp16 state values,
    #     with the new state rounded once
    yo, so = O.recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, s16.astype(np.float32), g, k_k.reshape(-1), k_a.reshape(-1),
                                            r_k, nw, nb, EPS)
    st = cu(s16)
    y, s_new = hb.fused_recurrent_output_prepare_raw(*dev, st, *par, eps=EPS)
    assert s_new.dtype == torch.float16 and torch.equal(st, cu(s16))  # out of place: the input state is untouched
    np.testing.assert_allclose(npf(s_new), so.astype(np.float16).astype(np.float32), atol=2e-3, rtol=2e-3)
    assert (npf(s_new) != so.astype(np.float16).astype(np.float32)).mean() < 0.02  # identical up to rare last-bit ties
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=2e-2, atol=2e-2)
    assert _cos_min(npf(y), yo) >= 0.9999
    # the reference's gate against the fp32-state result
    yo32, so32 = O.recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, s32, g, k_k.reshape(-1), k_a.reshape(-1), r_k, nw, nb, EPS)
    np.testing.assert_allclose(npf(s_new), so32, atol=3e-3, rtol=1e-2)
    assert _cos_min(npf(y), yo32) >= 0.999
    # (2) the extension's entry point: in place, dither phased by elapsed, elapsed advanced afterwards
    el = np.arange(B, dtype=np.int32) * 7 + 3
    yo16, so16 = O.native_fp16_recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, s16, g, k_k, k_a, r_k, nw, nb, el, EPS)
    st2, el_g = cu(s16), cu(el)
    y2 = hb.native_fp16_recurrent_output_prepare_raw(*dev, st2, cu(g), cu(k_k), cu(k_a), cu(r_k), cu(nw), cu(nb), el_g,
                                                     advance_elapsed=True, eps=EPS)
    assert np.array_equal(el_g.cpu().numpy(), el + 1)
    # against the restated reference kernel (fp16 arithmetic there, fp32 here): within a few fp16 ulps of the state
    np.testing.assert_allclose(npf(st2), so16.astype(np.float32), atol=3e-3, rtol=1e-2)
    assert _cos_min(npf(y2), yo16) >= 0.999
    np.testing.assert_allclose(npf(st2), so32, atol=3e-3, rtol=1e-2)
    assert _cos_min(npf(y2), yo32) >= 0.999
    # the prepared-input operator takes an fp16 state as well
    kkv = h(O.l2normalize_heads((k_raw.astype(np.float32) * k_k[None].astype(np.float32)).reshape(B, Hh * N), Hh, N).reshape(B, Hh, N))
    dec = np.exp(-0.606531 / (1 + np.exp(-w_raw.astype(np.float32)))).astype(np.float32)
    yp, sp = hb.fused_recurrent_output_prepare(cu(r), cu(dec), cu(k_raw), cu(v), cu(kkv), cu(a), cu(s16), cu(g), cu(r_k), cu(nw),
                                               cu(nb), eps=EPS)
    yop, sop = O.recurrent_output_prepare(r, dec, k_raw, v, kkv, a, s32, g, r_k, nw, nb, EPS)
    assert sp.dtype == torch.float16
    np.testing.assert_allclose(npf(sp), sop, atol=3e-3, rtol=1e-2)
    assert _cos_min(npf(yp), yop) >= 0.999
    with pytest.raises(ValueError):  # the plain update keeps the fp32 contract, as in the reference
        hb.fused_recurrent_update(cu(r), cu(dec), cu(k_raw), cu(v), cu(kkv), cu(a), cu(s16))


def test_dither_keeps_a_slowly_decaying_fp16_state_unbiased():
    """Pure decay (k = v = 0, kk * a = 0) by 0.99985 per step of a state of ones: round-to-nearest alone never changes
    a value near 1.0 (half an ulp is 2.4e-4), the dithered decay follows the fp32 trajectory on average."""
    B, Hh, steps = 2, 2, 256
    z = torch.zeros(B, Hh, N, device="cuda", dtype=torch.float16)
    one_p = lambda *s: torch.ones(*s, device="cuda", dtype=torch.float16)
    # decay = exp(-0.606531 * sigmoid(w_raw)) = 0.99985  ->  sigmoid = 2.473e-4  ->  w_raw = -8.305
    w_raw = torch.full((B, Hh, N), -8.305, device="cuda", dtype=torch.float16)
    decay = float(np.exp(-0.606531 / (1 + np.exp(8.305))))
    args = (z, w_raw, z, z, z)
    par = (z, one_p(Hh * N), one_p(Hh * N), z[0], one_p(Hh * N), z[0].reshape(-1))
    frozen = torch.ones(B, Hh, N, N, device="cuda", dtype=torch.float16)
    dith = frozen.clone()
    el = torch.zeros(B, device="cuda", dtype=torch.int32)
    for _ in range(steps):
        hb.fused_recurrent_output_prepare_raw(*args, frozen, *par, eps=EPS, new_state=frozen)
        hb.fused_recurrent_output_prepare_raw(*args, dith, *par, eps=EPS, new_state=dith, elapsed=el, advance_elapsed=True)
    assert float(frozen.float().mean()) == 1.0
    want = decay ** steps  # 0.9623
    assert abs(float(dith.float().mean()) - want) < 0.25 * (1 - want)
    assert int(el[0]) == steps


@pytest.mark.parametrize("B,T,Hh", [(2, 5, 2), (3, 40, 3)])
def test_sequence_lane(B, T, Hh):
    r, w, k, v, kk, a = wkv_inputs(B, T, Hh, N, seed=T + Hh)
    rng = np.random.default_rng(T)
    w_raw = h(rng.standard_normal((B, T, Hh, N)) - 1.0)
    w0 = h(0.5 * rng.standard_normal(Hh * N))
    s32 = (0.1 * rng.standard_normal((B, Hh, N, N))).astype(np.float32)
    s16 = s32.astype(np.float16)
    r, k, v, kk, a = (h(0.3 * x) if i in (0, 1, 2) else h(x) for i, x in enumerate((r, k, v, kk, a)))
    neg_kk, kka = h(-kk.astype(np.float32)), h(kk.astype(np.float32) * a.astype(np.float32))
    el = np.arange(B, dtype=np.int32) * 11
    for use_w0 in (False, True):
        yo, so = O.native_fp16_sequence(r, w_raw, k, v, neg_kk, kka, s16, el, w0 if use_w0 else None)
        st = cu(s16)
        y = hb.native_fp16_sequence(cu(r), cu(w_raw), cu(k), cu(v), cu(neg_kk), cu(kka), st, cu(el), w0=cu(w0) if use_w0 else None)
        np.testing.assert_allclose(npf(st), so.astype(np.float32), atol=3e-3, rtol=1e-2)
        assert rel_err(npf(y), yo.astype(np.float32)) < 2e-2
        # fp32 truth of the same recurrence (decay without dither)
        wv = w_raw.astype(np.float32) + (w0.astype(np.float32).reshape(1, 1, Hh, N) if use_w0 else 0)
        dec = np.exp(-0.606531 / (1 + np.exp(-wv))).astype(np.float32)
        yt, st_true = O.recurrent_scan(r, dec, k, v, kk, a, s32, hi=True)
        np.testing.assert_allclose(npf(st), st_true, atol=3e-3, rtol=1e-2)
        assert rel_err(npf(y), yt.astype(np.float32)) < 2e-2
    # the generic scans accept an fp16 state too (no dither): state in -> new state out, input untouched
    dec = np.exp(-0.606531 / (1 + np.exp(-w_raw.astype(np.float32)))).astype(np.float32)
    st = cu(s16)
    y2, s2 = hb.fused_recurrent_scan(cu(r), cu(dec), cu(k), cu(v), cu(kk), cu(a), st)
    yt, st_true = O.recurrent_scan(r, dec, k, v, kk, a, s16.astype(np.float32), hi=True)
    assert s2.dtype == torch.float16 and torch.equal(st, cu(s16))
    np.testing.assert_allclose(npf(s2), st_true.astype(np.float16).astype(np.float32), atol=2e-3, rtol=2e-3)
    assert rel_err(npf(y2), yt.astype(np.float32)) < 4e-3


def test_model_with_fp16_state_cache():
    """The tiny reference model in fp16 with state_dtype=float16: decode logits track the fp32-state model (cosine
    >= 0.999), the CUDA-graph replay equals the eager step bit for bit (the dither phase lives in the cache), prefill
    agrees with token-by-token decode, the cache halves its state bytes and carries the elapsed counters through
    clone / select_batch."""
    from tests.gpu_util import golden
    from tests.test_model_gpu import tiny_cfg
    g = golden("model_tiny.npz")
    sd = {k_[len("param::"):]: torch.from_numpy(v_) for k_, v_ in g.items() if k_.startswith("param::")}
    models = []
    for sdt in (torch.float32, torch.float16):
        m = hb.RWKV7ForCausalLM(tiny_cfg(), state_dtype=sdt)
        m.load_state_dict(sd)
        models.append(m.half().cuda().eval())
    m32, m16 = models
    ids = cu(g["ids"])
    B, T = ids.shape
    c32, c16e, c16g = m32.new_cache(B), m16.new_cache(B), m16.new_cache(B)
    assert c16e._state[0].dtype == torch.float16 and c16e._elapsed.dtype == torch.int32 and c32._elapsed is None
    for t in range(T):
        l32 = m32.rwkv7_forward_token(ids[:, t], c32, use_graph=False)
        le = m16.rwkv7_forward_token(ids[:, t], c16e, use_graph=False)
        lg = m16.rwkv7_forward_token(ids[:, t], c16g, use_graph=True)
        assert torch.equal(le, lg)
        assert _cos_min(npf(le), npf(l32)) >= 0.999
    assert int(c16e._elapsed[0]) == T and int(c16g._elapsed[1]) == T
    s32, s16 = npf(torch.stack(c32._state)), npf(torch.stack(c16e._state))
    np.testing.assert_allclose(s16, s32, atol=6e-3, rtol=2e-2)
    lp, cp = m16.rwkv7_prefill_native(ids, None)
    assert cp._state[0].dtype == torch.float16 and int(cp._elapsed[0]) == T
    assert _cos_min(npf(lp[:, -1]), npf(le)) >= 0.999
    c2 = c16e.clone().select_batch(torch.tensor([1], device="cuda"), inplace=False)
    assert tuple(c2._elapsed.shape) == (1,) and int(c2._elapsed[0]) == T and c2._state[0].dtype == torch.float16
    with pytest.raises(ValueError):  # an fp32 cache cannot be bound to the fp16-state model's graph
        m16.rwkv7_forward_token(ids[:, 0], c32, use_graph=True)
