"""CPU restatement (NumPy) of the RWKV-7 inference hot path of rwkv-rs/hf-adapter.

TEST INFRASTRUCTURE ONLY.  This module is the checker used by ``tests/``, by
``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``.  Nothing in the product package imports it: the product
path is the CUDA library and fails loudly without it.

Parity status: PINNED.  Every function below is checked against outputs of the
reference's own pure-torch path (``force_fallback=True`` operators and the eager
model) that were generated in a container where the reference imports, and
committed as fixtures under ``tests/golden/`` together with the generating
script ``tests/golden/make_golden.py``.

Numeric contract (the one the reference's fused kernels implement, e.g.
``rwkv7_hf/fused_recurrent_update.py:115-138``): inputs are taken in their
storage dtype (fp16/fp32), all arithmetic is fp32 (``float64`` when
``hi=True`` is passed, used to bound accumulation-order noise), outputs are
rounded once to the activation dtype, the recurrent state stays fp32.

Citations are ``file:line`` inside the reference project.
"""
from __future__ import annotations

import numpy as np

EXP_HALF = 0.606531  # rwkv7_hf/native.py:52 (the reference's constant, not exp(-0.5) exactly)


def _f(x, hi=False):
    return np.asarray(x, dtype=np.float64 if hi else np.float32)


def sigmoid(x):
    x = np.asarray(x)
    return (1.0 / (1.0 + np.exp(-x))).astype(x.dtype)


# --------------------------------------------------------------------------
# LayerNorm + token-shift mixes
# --------------------------------------------------------------------------

def layer_norm(x, weight, bias, eps=1e-5, hi=False):
    """LayerNorm over the last axis, biased variance (torch F.layer_norm)."""
    xf = _f(x, hi)
    mean = xf.mean(-1, keepdims=True)
    cen = xf - mean
    var = (cen * cen).mean(-1, keepdims=True)
    return cen / np.sqrt(var + eps) * _f(weight, hi) + _f(bias, hi)


def attn_norm_mix6_decode(x, previous, norm_w, norm_b, mixes, eps=1e-5, hi=False):
    """rwkv7_hf/fused_decode_norm_mix.py:38-86 (kernel) / :203-206 (fallback).

    h = LN(x); out_m = h + (previous - h) * mix_m for the six mixes in the
    order r,w,k,v,a,g; the new shift state is h.  Returns
    (six mixed arrays, new_previous), all rounded to x.dtype.
    """
    dt = np.asarray(x).dtype
    h = layer_norm(x, norm_w, norm_b, eps, hi)
    delta = _f(previous, hi) - h
    outs = tuple((h + delta * _f(m, hi).reshape(-1)).astype(dt) for m in mixes)
    return outs, h.astype(dt)


def ffn_add_norm_mix_decode(residual, attn_out, previous, norm_w, norm_b, mix, eps=1e-5, hi=False):
    """rwkv7_hf/fused_decode_norm_mix.py:88-119: x=res+attn; h=LN(x);
    mixed=h+(prev-h)*mix; prev<-h.  Returns (x, mixed, new_previous)."""
    dt = np.asarray(residual).dtype
    x = _f(residual, hi) + _f(attn_out, hi)
    h = layer_norm(x, norm_w, norm_b, eps, hi)
    mixed = h + (_f(previous, hi) - h) * _f(mix, hi).reshape(-1)
    return x.astype(dt), mixed.astype(dt), h.astype(dt)


def sequence_shift_mix(x, initial_prev, mixes, hi=False):
    """rwkv7_hf/fused_time_mix.py:136-301: x [B,T,D] already normalised;
    prev_t = x_{t-1} (initial_prev for t=0); out_m = x + (prev - x)*mix_m;
    next_state = x[:, -1]."""
    dt = np.asarray(x).dtype
    xf = _f(x, hi)
    prev = np.concatenate([_f(initial_prev, hi)[:, None, :], xf[:, :-1]], axis=1)
    d = prev - xf
    outs = tuple((xf + d * _f(m, hi).reshape(-1)).astype(dt) for m in mixes)
    return outs, np.asarray(x)[:, -1].copy()


# --------------------------------------------------------------------------
# LoRA group
# --------------------------------------------------------------------------

def _lin(x, w, b=None):
    y = x @ w.T
    if b is not None:
        y = y + b
    return y


def wavg_lora(xw, xa, xg, xv, downs, ups, biases, hi=False):
    """rwkv7_hf/fused_lora.py:796-803.  Returns raw w, PRE-sigmoid a, g and
    POST-sigmoid v_gate (v parts may be None: then v_gate is None).
    downs/ups/biases are (w, a, g, v) tuples; weights are [out,in]."""
    dt = np.asarray(xw).dtype
    f = lambda t: None if t is None else _f(t, hi)
    wd, ad, gd, vd = (f(t) for t in downs)
    wu, au, gu, vu = (f(t) for t in ups)
    wb, ab, gb, vb = (f(t) for t in biases)
    # The reference rounds every Linear output to the activation dtype.
    rd = lambda t: t.astype(dt).astype(t.dtype)
    wh = rd(np.tanh(rd(_lin(_f(xw, hi), wd))))
    ah = rd(_lin(_f(xa, hi), ad))
    gh = rd(sigmoid(rd(_lin(_f(xg, hi), gd))))
    w_out = _lin(wh, wu, wb).astype(dt)
    a_out = _lin(ah, au, ab).astype(dt)
    g_out = _lin(gh, gu, gb).astype(dt)
    v_gate = None
    if vd is not None:
        vh = rd(_lin(_f(xv, hi), vd))
        v_gate = sigmoid(rd(_lin(vh, vu, vb))).astype(dt)
    return w_out, a_out, g_out, v_gate


# --------------------------------------------------------------------------
# State prep / output prep
# --------------------------------------------------------------------------

def l2normalize_heads(x, H, N, eps=1e-12):
    """F.normalize(p=2, dim=-1) per head: x / max(||x||, eps)
    (rwkv7_hf/native.py:215-219)."""
    shp = x.shape
    xh = x.reshape(shp[:-1] + (H, N))
    nrm = np.sqrt((xh * xh).sum(-1, keepdims=True))
    return (xh / np.maximum(nrm, eps)).reshape(shp)


def prefill_state_prep(w_raw, k_raw, v_raw, a, k_k, k_a, H, N, v_first=None, v_gate=None,
                       a_is_raw=False, v_gate_is_raw=False, log_decay=False, hi=False):
    """rwkv7_hf/fused_prefill.py:256-279.  Returns (w fp32, k, v, kk)."""
    dt = np.asarray(k_raw).dtype
    af = _f(a, hi)
    if a_is_raw:
        af = sigmoid(af)
    kf = _f(k_raw, hi)
    kk = l2normalize_heads(kf * _f(k_k, hi).reshape(-1), H, N)
    k_out = kf * (1 + (af - 1) * _f(k_a, hi).reshape(-1))
    vf = _f(v_raw, hi)
    if v_first is not None and v_gate is not None:
        vg = _f(v_gate, hi)
        if v_gate_is_raw:
            vg = sigmoid(vg)
        vf = vf + (_f(v_first, hi) - vf) * vg
    w_log = -EXP_HALF * sigmoid(_f(w_raw, hi))
    w_out = w_log if log_decay else np.exp(w_log)
    return w_out.astype(np.float32), k_out.astype(dt), vf.astype(dt), kk.astype(dt)


def prefill_kv_kk_prep(k_raw, v_raw, a, k_k, k_a, H, N, v_first=None, v_gate=None, hi=False):
    """rwkv7_hf/fused_prefill.py:324-392: state prep without the decay.  Returns (k, v, kk)."""
    _, k, v, kk = prefill_state_prep(np.zeros_like(k_raw), k_raw, v_raw, a, k_k, k_a, H, N, v_first, v_gate, hi=hi)
    return k, v, kk


def group_norm_heads(y, H, N, weight, bias, eps):
    """GroupNorm with H groups over [.., H*N], biased variance
    (rwkv7_hf/fused_recurrent_update.py:136-141)."""
    shp = y.shape
    yh = y.reshape(shp[:-1] + (H, N))
    mean = yh.mean(-1, keepdims=True)
    cen = yh - mean
    var = (cen * cen).mean(-1, keepdims=True)
    out = (cen / np.sqrt(var + eps)).reshape(shp)
    return out * weight.reshape(-1) + bias.reshape(-1)


def attn_output_prepare(recurrent, r, k, v, g, r_k, gn_w, gn_b, H, N, eps, hi=False):
    """rwkv7_hf/fused_output.py:190 / fused_recurrent_update.py:903-911:
    (GroupNorm(y) + (sum_n r k r_k) v) * g over [rows, H*N]."""
    dt = np.asarray(r).dtype
    y = _f(recurrent, hi)
    rows = y.shape[:-1]
    normed = group_norm_heads(y, H, N, _f(gn_w, hi), _f(gn_b, hi), eps)
    rf, kf, vf = (_f(t, hi).reshape(rows + (H, N)) for t in (r, k, v))
    corr = (rf * kf * _f(r_k, hi).reshape(H, N)).sum(-1, keepdims=True) * vf
    out = (normed + corr.reshape(y.shape)) * _f(g, hi)
    return out.astype(dt)


def attn_output_project(recurrent, r, k, v, g, r_k, gn_w, gn_b, o_w, o_b, H, N, eps, hi=False):
    """rwkv7_hf/fused_output.py:278-394: output prep followed by o_proj (dense [out, H*N] weight, optional bias)."""
    dt = np.asarray(r).dtype
    prepared = attn_output_prepare(recurrent, r, k, v, g, r_k, gn_w, gn_b, H, N, eps, hi)
    y = _f(prepared, hi) @ _f(o_w, hi).T
    if o_b is not None:
        y = y + _f(o_b, hi)
    return y.astype(dt)


def ffn(x, prev, mix, key_w, value_w, hi=False):
    """rwkv7_hf/fused_ffn.py:394-486 (one token) and :245-376 (sequence: prev is the state before the first token).
    k = x + (shift(x) - x) * mix; out = value(relu(key(k))^2).  Returns (out, next_state = last x)."""
    dt = np.asarray(x).dtype
    xf = _f(x, hi)
    if xf.ndim == 3:
        shifted = np.concatenate([_f(prev, hi)[:, None], xf[:, :-1]], axis=1)
        nxt = np.asarray(x)[:, -1]
    else:
        shifted = _f(prev, hi)
        nxt = np.asarray(x)
    kx = (xf + (shifted - xf) * _f(mix, hi).reshape(-1)).astype(dt)
    mid = (np.maximum(_f(kx, hi) @ _f(key_w, hi).T, 0).astype(dt).astype(xf.dtype) ** 2).astype(dt)
    out = (_f(mid, hi) @ _f(value_w, hi).T).astype(dt)
    return out, nxt


# --------------------------------------------------------------------------
# WKV-7 recurrence
# --------------------------------------------------------------------------

def recurrent_update(r, w, k, v, kk, a, state, hi=False):
    """One token.  rwkv7_hf/fused_recurrent_update.py:757-783 (math) in the
    rank-1 form of the kernels (:125-131):

        sa[i]   = sum_m S[i,m] kk[m]
        S'[i,j] = S[i,j] w[j] + v[i] k[j] - sa[i] kk[j] a[j]
        y[i]    = sum_j S'[i,j] r[j]

    Vectors are [B,H,N]; state [B,H,N,N] (rows = value index, cols = key
    index).  Returns (y in r.dtype, new state fp32)."""
    dt = np.asarray(r).dtype
    S = _f(state, hi)
    rf, wf, kf, vf, kkf, af = (_f(t, hi) for t in (r, w, k, v, kk, a))
    sa = np.einsum("bhij,bhj->bhi", S, kkf)
    Sn = S * wf[:, :, None, :] + vf[..., :, None] * kf[..., None, :] \
        - sa[..., :, None] * (kkf * af)[..., None, :]
    y = np.einsum("bhij,bhj->bhi", Sn, rf)
    return y.astype(dt), Sn.astype(np.float32) if not hi else Sn


def recurrent_output_prepare(r, w, k, v, kk, a, state, g, r_k, gn_w, gn_b, eps, hi=False):
    """rwkv7_hf/fused_recurrent_update.py:870-915 / kernel :86-152.  The
    kernel keeps y in fp32 through the GroupNorm; so does this."""
    dt = np.asarray(r).dtype
    B, H, N, _ = state.shape
    S = _f(state, hi)
    rf, wf, kf, vf, kkf, af, gf = (_f(t, hi).reshape(B, H, N) for t in (r, w, k, v, kk, a, g))
    sa = np.einsum("bhij,bhj->bhi", S, kkf)
    Sn = S * wf[:, :, None, :] + vf[..., :, None] * kf[..., None, :] \
        - sa[..., :, None] * (kkf * af)[..., None, :]
    y = np.einsum("bhij,bhj->bhi", Sn, rf)
    mean = y.mean(-1, keepdims=True)
    cen = y - mean
    var = (cen * cen).mean(-1, keepdims=True)
    normed = cen / np.sqrt(var + eps)
    corr = (rf * kf * _f(r_k, hi).reshape(1, H, N)).sum(-1, keepdims=True)
    out = (normed * _f(gn_w, hi).reshape(1, H, N) + _f(gn_b, hi).reshape(1, H, N) + corr * vf) * gf
    return out.astype(dt), Sn.astype(np.float32)


def recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, state, g, k_k, k_a, r_k, gn_w, gn_b, eps, hi=False):
    """rwkv7_hf/fused_recurrent_update.py:154-229: decay, kk-normalise and
    k-adjust computed in fp32 from raw w/k, then the step above."""
    B, H, N, _ = state.shape
    kr = _f(k_raw, hi).reshape(B, H, N)
    af = _f(a, hi).reshape(B, H, N)
    kk = l2normalize_heads(kr * _f(k_k, hi).reshape(1, H, N), 1, N)
    k = kr * (1.0 + (af - 1.0) * _f(k_a, hi).reshape(1, H, N))
    w = np.exp(-EXP_HALF * sigmoid(_f(w_raw, hi).reshape(B, H, N)))
    dt = np.asarray(r).dtype
    out, Sn = recurrent_output_prepare(_f(r, hi).reshape(B, H, N), w, k, _f(v, hi).reshape(B, H, N), kk, af,
                                       state, _f(g, hi).reshape(B, H, N), r_k, gn_w, gn_b, eps, hi)
    return out.astype(dt), Sn


def recurrent_scan(r, w, k, v, kk, a, state, hi=False):
    """T sequential steps.  rwkv7_hf/fused_recurrent_update.py:800-867.
    Inputs [B,T,H,N]; returns (y [B,T,H,N] in r.dtype, final state)."""
    dt = np.asarray(r).dtype
    B, T, H, N = r.shape
    S = _f(state, hi).copy()
    rf, wf, kf, vf, kkf, af = (_f(t, hi) for t in (r, w, k, v, kk, a))
    bq = kkf * af
    y = np.empty((B, T, H, N), dtype=S.dtype)
    for t in range(T):
        sa = np.einsum("bhij,bhj->bhi", S, kkf[:, t])
        S = S * wf[:, t, :, None, :] + vf[:, t, :, :, None] * kf[:, t, :, None, :] \
            - sa[..., :, None] * bq[:, t, :, None, :]
        y[:, t] = np.einsum("bhij,bhj->bhi", S, rf[:, t])
    return y.astype(dt), S.astype(np.float32)


def recurrent_scan_state_prep(r, w_raw, k_raw, v_raw, a, state, k_k, k_a, H, N, v_first=None, v_gate=None, hi=False):
    """rwkv7_hf/fused_recurrent_update.py:1541-1650: state prep folded into the scan.
    Inputs [B,T,H,N]; returns (y, final state, adjusted k, interpolated v)."""
    shp = np.asarray(r).shape
    flat = lambda t: None if t is None else np.asarray(t).reshape(shp[0], shp[1], H * N)
    w, k, v, kk = prefill_state_prep(flat(w_raw), flat(k_raw), flat(v_raw), flat(a), k_k, k_a, H, N, flat(v_first),
                                     flat(v_gate), hi=hi)
    y, S = recurrent_scan(r, w.reshape(shp), k.reshape(shp), v.reshape(shp), kk.reshape(shp), a, state, hi)
    return y, S, k.reshape(shp), v.reshape(shp)


def chunk_scan(r, w, k, v, kk, a, state, chunk=16):
    """Chunked DPLR / WY form of the same scan (float64 throughout), used to
    check chunk-size independence.  Algorithm of
    rwkv7_hf/self_chunk_rwkv7.py:33-134 restated in the native [V,K] state
    orientation (see also rwkv7_hf/dplr_prefill.py:221-311):

      per chunk with cumulative decays P_t = prod_{s<=t} w_s (inclusive) and
      E_t = P_t / w_t (exclusive), a~ = -kk, b~ = kk*a:
        A_ab[t,s] = sum_n a~_t E_t / P_s b~_s   (t>s)
        A_ak[t,s] = sum_n a~_t E_t / P_s k_s    (t>s)
        (I - A_ab) U = A_ak V + (a~ E) S0^T     -> U rows u_t = S_{t-1} a~_t
        y_t = S0 (r_t P_t) + sum_{s<=t} [ (r_t P_t/P_s . k_s) v_s + (r_t P_t/P_s . b~_s) u_s ]
        S_C = S0 diag(P_C) + sum_s ( v_s (k_s P_C/P_s)^T + u_s (b~_s P_C/P_s)^T )
    """
    dt = np.asarray(r).dtype
    B, T, H, N = r.shape
    S = np.asarray(state, dtype=np.float64).copy()
    f = lambda t: np.asarray(t, dtype=np.float64).transpose(0, 2, 1, 3)  # [B,H,T,N]
    rf, wf, kf, vf, kkf, af = (f(t) for t in (r, w, k, v, kk, a))
    at, bt = -kkf, kkf * af
    y = np.empty((B, H, T, N))
    for c0 in range(0, T, chunk):
        c1 = min(T, c0 + chunk)
        C = c1 - c0
        sl = slice(c0, c1)
        lw = np.log(wf[:, :, sl])
        gi = np.cumsum(lw, axis=2)
        ge = gi - lw
        P, E = np.exp(gi), np.exp(ge)
        invP = np.exp(-gi)
        gl = gi[:, :, -1:, :]
        strict = np.tril(np.ones((C, C)), -1)
        incl = np.tril(np.ones((C, C)))
        aE = at[:, :, sl] * E
        A_ab = np.einsum("bhtn,bhsn->bhts", aE, bt[:, :, sl] * invP) * strict
        A_ak = np.einsum("bhtn,bhsn->bhts", aE, kf[:, :, sl] * invP) * strict
        rhs = np.einsum("bhts,bhsi->bhti", A_ak, vf[:, :, sl]) + np.einsum("bhtn,bhin->bhti", aE, S)
        U = np.linalg.solve(np.eye(C) - A_ab, rhs)  # [B,H,C,N(value idx)]
        rP = rf[:, :, sl] * P
        A_qk = np.einsum("bhtn,bhsn->bhts", rP, kf[:, :, sl] * invP) * incl
        A_qb = np.einsum("bhtn,bhsn->bhts", rP, bt[:, :, sl] * invP) * incl
        y[:, :, sl] = np.einsum("bhtn,bhin->bhti", rP, S) \
            + np.einsum("bhts,bhsi->bhti", A_qk, vf[:, :, sl]) \
            + np.einsum("bhts,bhsi->bhti", A_qb, U)
        dec = np.exp(gl - gi)
        S = S * np.exp(gl)[:, :, 0, None, :] \
            + np.einsum("bhsi,bhsn->bhin", vf[:, :, sl], kf[:, :, sl] * dec) \
            + np.einsum("bhsi,bhsn->bhin", U, bt[:, :, sl] * dec)
    return y.transpose(0, 2, 1, 3).astype(dt), S.astype(np.float32)


# --------------------------------------------------------------------------
# Quantisation formats and integer GEMMs
# --------------------------------------------------------------------------

def _round_half_even(x):
    return np.rint(x)


def quantize_w8_row(weight, scale_dtype=np.float16):
    """rwkv7_hf/sm70_quant.py:485-489: s=max(amax_row/127,1e-6) (fp32),
    q=round_half_even(w/s) clamp +-127; scale stored in the weight dtype."""
    w = np.asarray(weight, dtype=np.float32)
    s = np.maximum(np.abs(w).max(1) / np.float32(127), np.float32(1e-6)).astype(np.float32)
    q = np.clip(_round_half_even(w / s[:, None]), -127, 127).astype(np.int8)
    return q, s.astype(scale_dtype)


def quantize_w4_groupwise(weight, group_size=128, scale_dtype=np.float16):
    """rwkv7_hf/sm70_quant.py:502-519: symmetric, q in [1,15] (zero-point 8),
    packed [out, in/2] with the low nibble = even k; scales [out, in/group]."""
    w = np.asarray(weight, dtype=np.float32)
    O, K = w.shape
    g = w.reshape(O, K // group_size, group_size)
    s = np.maximum(np.abs(g).max(2) / np.float32(7), np.float32(1e-6)).astype(np.float32)
    q = (np.clip(_round_half_even(g / s[:, :, None]), -7, 7).astype(np.int16) + 8).reshape(O, K)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return packed, s.astype(scale_dtype)


def unpack_w4(packed):
    """[out, in/2] u8 -> [out, in] int (0..15), low nibble first."""
    O, K2 = packed.shape
    q = np.empty((O, K2 * 2), dtype=np.int16)
    q[:, 0::2] = packed & 15
    q[:, 1::2] = packed >> 4
    return q


def dequant_w4_groupwise(packed, scales, zeros=None, group_size=128, dtype=np.float16):
    """rwkv7_hf/sm70_quant.py:598-606: W = (nibble - zero) * scale evaluated in
    the activation dtype (zero = 8 when no zero-point tensor is given)."""
    q = unpack_w4(packed).astype(np.float32)
    z = np.float32(8) if zeros is None else np.repeat(np.asarray(zeros, np.float32), group_size, axis=1)
    s = np.repeat(np.asarray(scales).astype(dtype).astype(np.float32), group_size, axis=1)
    return ((q - z).astype(dtype).astype(np.float32) * s).astype(dtype)


def w4_groupwise_linear(x, packed, scales, zeros=None, group_size=128, hi=False):
    """rwkv7_hf/sm70_quant.py:579-610 CPU branch: materialise the activation
    dtype weight then F.linear (fp32 accumulate, one rounding at the end)."""
    dt = np.asarray(x).dtype
    W = dequant_w4_groupwise(packed, scales, zeros, group_size, dtype=dt)
    return (_f(x, hi) @ _f(W, hi).T).astype(dt)


def w8_linear(x, q, s, hi=False):
    """rwkv7_hf/sm70_quant.py:522-531 CPU branch: F.linear(x, q.to(dtype)*s)."""
    dt = np.asarray(x).dtype
    W = (q.astype(dt).astype(np.float32) * np.asarray(s).astype(dt).astype(np.float32)[:, None]).astype(dt)
    return (_f(x, hi) @ _f(W, hi).T).astype(dt)


def quantize_weight_per_channel_int8(weight):
    """rwkv7_hf/native_quant_a8w8.py:312-320: returns (q^T [in,out] int8,
    scale [out] fp32), s=max(amax/127,1e-5)."""
    w = np.asarray(weight, dtype=np.float32)
    s = np.maximum(np.abs(w).max(1) / np.float32(127), np.float32(1e-5)).astype(np.float32)
    q = np.clip(_round_half_even(w / s[:, None]), -127, 127).astype(np.int8)
    return np.ascontiguousarray(q.T), s


def dynamic_a8_quant(x):
    """rwkv7_hf/native_quant_a8w8.py:134-164 with IEEE fp32 division:
    per row s=max(amax/127,1e-5); q=clamp(round_half_away(x/s),+-127)."""
    xf = np.asarray(x, dtype=np.float32)
    s = np.maximum(np.abs(xf).max(-1) / np.float32(127), np.float32(1e-5)).astype(np.float32)
    sc = (xf / s[..., None]).astype(np.float32)
    q = np.where(sc >= 0, np.floor(sc + np.float32(0.5)), np.ceil(sc - np.float32(0.5)))
    return np.clip(q, -127, 127).astype(np.int8), s


def int8_gemm_i32(qa, qw_t, exact_int64=False):
    """Exact integer truth of torch._int_mm (native_quant_a8w8.py:413): [rows,K] int8 x [K,out] int8 -> int32.
    Computed in float64 through BLAS when every partial sum provably stays below 2^53 (|q| <= 128, so K * 2^14 < 2^53:
    products and sums of integers of that size are exact in float64), which is hundreds of times faster than NumPy's
    int64 matmul at projection sizes; ``exact_int64`` (or a longer K) takes the int64 route.  The two agree bit for
    bit (tests/test_oracle_golden.py)."""
    K = int(qa.shape[-1])
    if exact_int64 or K * (1 << 14) >= (1 << 53):
        acc = qa.astype(np.int64) @ qw_t.astype(np.int64)
    else:
        acc = np.rint(qa.astype(np.float64) @ qw_t.astype(np.float64)).astype(np.int64)
    assert np.abs(acc).max(initial=0) < 2 ** 31
    return acc.astype(np.int32)


def a8w8_linear(x, q_weight_t, weight_scale, bias=None, residual=None):
    """rwkv7_hf/native_quant_a8w8.py:398-432 + dequant kernel :166-188:
    out = fp32(acc) * s_row * s_col (+bias) (+residual), rounded to x.dtype.
    Returns (out, acc_i32, q_act, s_act)."""
    dt = np.asarray(x).dtype
    qa, sa = dynamic_a8_quant(x)
    acc = int8_gemm_i32(qa, q_weight_t)
    out = acc.astype(np.float32) * sa[:, None] * np.asarray(weight_scale, np.float32)[None, :]
    if bias is not None:
        out = out + np.asarray(bias, np.float32)
    if residual is not None:
        out = out + np.asarray(residual, np.float32)
    return out.astype(dt), acc, qa, sa


def a8w8_relu2_requant(acc, sa, sw):
    """rwkv7_hf/native_quant_a8w8.py:189-232: dequant, fp16 round, relu^2,
    fp16 round, per-row requantise.  Returns (q int8, scale fp32)."""
    pre = (acc.astype(np.float32) * sa[:, None] * np.asarray(sw, np.float32)[None, :])
    pre = pre.astype(np.float16).astype(np.float32)
    act = np.maximum(pre, 0)
    act = (act * act).astype(np.float16).astype(np.float32)
    return dynamic_a8_quant(act)


def quantize_mm8(weight):
    """fp16i8 affine format, rwkv7_hf/native_quant_mm8.py:62-97.  ``weight``
    is the transposed Linear weight [in(K), out(M)] in fp32.  Returns
    (w_u8 [K,M], mx [M], rx [M], my [K,1], ry [K,1]) in fp32 (callers store
    fp16)."""
    w = np.asarray(weight, dtype=np.float32).copy()
    K, M = w.shape
    if K > M:
        my = w.min(1, keepdims=True); w = w - my
        mx = w.min(0); w = w - mx
    else:
        mx = w.min(0); w = w - mx
        my = w.min(1, keepdims=True); w = w - my
    rx = np.maximum(w.max(0), np.float32(1e-8)); w = w / rx
    ry = np.maximum(w.max(1, keepdims=True), np.float32(1e-8)); w = w / ry
    u8 = np.clip(np.floor(w * 256), 0, 255).astype(np.uint8)
    return u8, mx, rx / 16, my, ry / 16


def mm8_matmul(x, w_u8, mx, rx, my, ry, hi=False):
    """rwkv7_hf/native_quant_mm8.py:100-105 / kernel :148-208:
    y[m] = sum_k x[k]((u8+0.5) ry[k] rx[m] + my[k] + mx[m]), fp32 accumulate."""
    dt = np.asarray(x).dtype
    W = (w_u8.astype(np.float32) + 0.5) * _f(ry, hi).reshape(-1, 1) * _f(rx, hi).reshape(1, -1) \
        + _f(my, hi).reshape(-1, 1) + _f(mx, hi).reshape(1, -1)
    return (_f(x, hi) @ W).astype(dt)


def _ops_in(dtype, q, ry, rx, my, mx):
    """(q + 0.5) * ry * rx + my + mx with every operation rounded to ``dtype``, the order of dequantize_mm8 /
    dequantize_mm4 (rwkv7_hf/native_quant_mm8.py:100-107, native_quant_mm4.py:111-125)."""
    t = np.dtype(dtype).type
    v = (q.astype(dtype) + t(0.5)).astype(dtype)
    v = (v * np.asarray(ry, dtype).reshape(-1, 1)).astype(dtype)
    v = (v * np.asarray(rx, dtype).reshape(1, -1)).astype(dtype)
    v = (v + np.asarray(my, dtype).reshape(-1, 1)).astype(dtype)
    return (v + np.asarray(mx, dtype).reshape(1, -1)).astype(dtype)


def dequantize_mm8(w_u8, mx, rx, my, ry, dtype=np.float16):
    return _ops_in(dtype, w_u8, ry, rx, my, mx)


def quantize_mm4(weight, out_dtype=np.float16):
    """4-bit affine format, rwkv7_hf/native_quant_mm4.py:77-108.  ``weight`` [K, M] (transposed Linear weight).
    Returns (packed [K, Mp/2] u8, mx [Mp], rx_s [Mp], my [K,1], ry_s [K,1], M, Mp)."""
    w = np.asarray(weight).astype(np.float32)
    K, M = w.shape
    if M % 2:
        w = np.pad(w, ((0, 0), (0, 1)))
    Mp = w.shape[1]
    if K > Mp:
        my = w.min(1, keepdims=True); w = w - my
        mx = w.min(0); w = w - mx
    else:
        mx = w.min(0); w = w - mx
        my = w.min(1, keepdims=True); w = w - my
    rx = np.maximum(w.max(0), np.float32(1e-8)); w = w / rx
    ry = np.maximum(w.max(1, keepdims=True), np.float32(1e-8)); w = w / ry
    u4 = np.clip(np.floor(w * np.float32(16)), 0, 15).astype(np.uint8)
    packed = (u4[:, 0::2] | (u4[:, 1::2] << 4)).astype(np.uint8)
    od = np.dtype(out_dtype)
    return packed, mx.astype(od), (rx / np.float32(4)).astype(od), my.astype(od), (ry / np.float32(4)).astype(od), M, Mp


def unpack_mm4(packed):
    u4 = np.empty((packed.shape[0], packed.shape[1] * 2), np.uint8)
    u4[:, 0::2] = packed & 15
    u4[:, 1::2] = packed >> 4
    return u4


def dequantize_mm4(packed, mx, rx_s, my, ry_s, m_orig, dtype=np.float16):
    return _ops_in(dtype, unpack_mm4(packed), ry_s, rx_s, my, mx)[:, :m_orig]


def mm4_matmul(x, packed, mx, rx_s, my, ry_s, m_orig, hi=False):
    """y = x @ W with W the affine 4-bit weight, fp32 accumulate (the fused kernel's arithmetic,
    rwkv7_hf/native_quant_mm4.py:150-215)."""
    dt = np.asarray(x).dtype
    W = (unpack_mm4(packed).astype(np.float32) + 0.5) * _f(ry_s, hi).reshape(-1, 1) * _f(rx_s, hi).reshape(1, -1) \
        + _f(my, hi).reshape(-1, 1) + _f(mx, hi).reshape(1, -1)
    return (_f(x, hi) @ W[:, :m_orig]).astype(dt)


def a8w8_ffn(x, up_q_t, up_s, down_q_t, down_s, residual, up_bias=None, down_bias=None):
    """rwkv7_hf/native_quant_a8w8.py:436-524: up GEMM, relu^2 + requantise at the boundary, down GEMM + residual.
    The reference's fused path is GPU-only (Triton + torch._int_mm); this restatement follows its kernels line by
    line and is pinned against the reference's own CPU composition of the same FFN (a8w8_linear -> relu^2 ->
    a8w8_linear + residual on the dequantised weights, fixture a8w8_ffn.npz) at the reference's gate for the A8
    approximation, cosine >= 0.999 (tests/test_native_quant_a8w8.py:63,92)."""
    qa, sa = dynamic_a8_quant(x)
    acc = int8_gemm_i32(qa, up_q_t)
    pre = acc.astype(np.float32) * sa[:, None] * np.asarray(up_s, np.float32)[None, :]
    if up_bias is not None:
        pre = pre + np.asarray(up_bias, np.float32)
    pre = pre.astype(np.float16).astype(np.float32)
    act = np.maximum(pre, 0)
    act = (act * act).astype(np.float16).astype(np.float32)
    qh, sh = dynamic_a8_quant(act)
    acc2 = int8_gemm_i32(qh, down_q_t)
    y = acc2.astype(np.float32) * sh[:, None] * np.asarray(down_s, np.float32)[None, :]
    if down_bias is not None:
        y = y + np.asarray(down_bias, np.float32)
    y = y + np.asarray(residual, np.float32)
    return y.astype(np.asarray(x).dtype), qh, sh


# --------------------------------------------------------------------------
# Whole token step / model (per-layer parameter dict, see tests/golden)
# --------------------------------------------------------------------------

def linear_op(x, op, hi=False):
    """A projection operand: dense [out,in] array, or a dict describing one of
    the quantised formats (keys: kind in {'w4g','w8','a8w8'})."""
    dt = np.asarray(x).dtype
    if callable(op):  # e.g. a sharded projection followed by a cross-rank sum (tensor-parallel tests)
        return op(x)
    if isinstance(op, dict):
        kind = op["kind"]
        if kind == "w4g":
            return w4_groupwise_linear(x, op["packed"], op["scales"], op.get("zeros"), op.get("group", 128), hi)
        if kind == "w8":
            return w8_linear(x, op["q"], op["s"], hi)
        if kind == "a8w8":
            return a8w8_linear(x, op["q_t"], op["s"])[0]
        if kind == "mm8":
            return mm8_matmul(x, op["u8"], op["mx"], op["rx"], op["my"], op["ry"], hi)
        if kind == "mm4":
            return mm4_matmul(x, op["packed"], op["mx"], op["rx"], op["my"], op["ry"], op["m"], hi)
        raise ValueError(kind)
    return (_f(x, hi) @ _f(op, hi).T).astype(dt)


def block_step(p, layer_id, x, xpa, xpf, v_first, state, H, N, hi=False):
    """One layer, one token for a batch: rwkv7_hf/native.py:390-419 with
    attn_step_batched (:180-272) and ffn_step_batched (:275-280).  Rounding
    points follow the fused decode path (fp32 inside each fused operator,
    activation dtype between operators).  ``p`` is a dict of arrays named as
    in the reference pack tuple (rwkv7_hf/native_jit_packing.py:13-58)."""
    dt = np.asarray(x).dtype
    rd = lambda t: np.asarray(t).astype(dt)
    if layer_id == 0 and p.get("pre_w") is not None:
        x = rd(layer_norm(x, p["pre_w"], p["pre_b"], 1e-5, hi))
    (xr, xw, xk, xv, xa, xg), xpa_new = attn_norm_mix6_decode(
        x, xpa, p["attn_w"], p["attn_b"], [p[n] for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")], 1e-5, hi)
    r = linear_op(xr, p["Rw"], hi)
    k_raw = linear_op(xk, p["Kw"], hi)
    v = linear_op(xv, p["Vw"], hi)
    has_v = layer_id != 0
    w_raw, a_pre, g, v_gate = wavg_lora(
        xw, xa, xg, xv if has_v else None,
        (p["w1"], p["a1"], p["g1"], p["v1"] if has_v else None),
        (p["w2"], p["a2"], p["g2"], p["v2"] if has_v else None),
        (p["w0"], p["a0"], None, p["v0"] if has_v else None), hi)
    a = rd(sigmoid(_f(a_pre, hi)))
    if has_v:
        v = rd(_f(v, hi) + (_f(v_first, hi) - _f(v, hi)) * _f(v_gate, hi))
        v_first_new = v_first
    else:
        v_first_new = v
    out, state_new = recurrent_output_prepare_raw(
        r, w_raw, k_raw, v, a, state, g, p["k_k"], p["k_a"], p["r_k"], p["gn_w"], p["gn_b"], N * 1e-5, hi)
    B = x.shape[0]
    attn = linear_op(out.reshape(B, H * N), p["Ow"], hi)
    x2, mixed, xpf_new = ffn_add_norm_mix_decode(x, attn, xpf, p["ffn_w"], p["ffn_b"], p["fx_k"], 1e-5, hi)
    kx = linear_op(mixed, p["fK"], hi)
    kf = np.maximum(_f(kx, hi), 0)
    hidden = rd(kf * kf)
    f = linear_op(hidden, p["fV"], hi)
    x3 = rd(_f(x2, hi) + _f(f, hi))
    return x3, xpa_new, xpf_new, v_first_new, state_new


def model_step(params, token_ids, cache, H, N, hi=False):
    """Embedding -> L x block_step -> final LayerNorm -> head
    (rwkv7_hf/native.py:444-452).  ``cache`` = dict(state[L], xpa[L], xpf[L],
    v_first); updated in place.  Returns logits [B,V] in the embedding dtype."""
    x = params["emb"][np.asarray(token_ids).reshape(-1)]
    dt = x.dtype
    v_first = cache["v_first"]
    for i, p in enumerate(params["layers"]):
        x, cache["xpa"][i], cache["xpf"][i], v_first, cache["state"][i] = block_step(
            p, i, x, cache["xpa"][i], cache["xpf"][i], v_first, cache["state"][i], H, N, hi)
    cache["v_first"] = v_first
    xn = layer_norm(x, params["norm_w"], params["norm_b"], 1e-5, hi).astype(dt)
    return linear_op(xn, params["head"], hi)


def new_cache(L, B, D, H, N, dtype):
    return dict(state=[np.zeros((B, H, N, N), np.float32) for _ in range(L)],
                xpa=[np.zeros((B, D), dtype) for _ in range(L)],
                xpf=[np.zeros((B, D), dtype) for _ in range(L)],
                v_first=np.zeros((B, H * N), dtype))


# --------------------------------------------------------------------------
# FP16-state lane (rwkv7_hf/native_wkv_fp16.py).  The reference's implementation of this lane is a CUDA extension
# without a CPU route, so these restatements follow its kernels instruction by instruction (every __hfma2 / __hadd
# rounds to fp16 once) but cannot be checked against reference outputs here: parity of this lane is pinned only
# through the reference's own gate for it, agreement with the fp32-state operators within atol 3e-3 / rtol 1e-2 on
# the state and cosine >= 0.999 on the outputs (tests/test_fused_recurrent_output_raw.py:44-141).  exp2f is exact
# here; the extension is built with --use_fast_math.
# --------------------------------------------------------------------------
_H = np.float16


def _hfma(a, b, c):
    """__hfma: a*b + c with one rounding to fp16 (the product of two halves is exact in float64)."""
    return (np.asarray(a, np.float64) * np.asarray(b, np.float64) + np.asarray(c, np.float64)).astype(_H)


def _hadd(a, b):
    return (np.asarray(a, np.float64) + np.asarray(b, np.float64)).astype(_H)


def rotator1(x):
    """native_wkv_fp16.py:118-121: 2^-41 * int32(2654435769 * uint32(x))."""
    bits = (np.asarray(x, np.int64).astype(np.uint64) * np.uint64(2654435769)) & np.uint64(0xFFFFFFFF)
    return np.float32(4.547473508864641e-13) * bits.astype(np.uint32).view(np.int32).astype(np.float32)


def w_delta(w_raw, phase, w0=None):
    """native_wkv_fp16.py:123-139: fp16(exp2(-0.875.../(1+exp2(-1.4427 w))) - 1 + rotator1(phase)), i.e. decay - 1
    plus the dither; ``w0`` is added to the raw value first when given."""
    w = np.asarray(w_raw, np.float32)
    if w0 is not None:
        w = w + np.asarray(w0, np.float32)
    d = np.exp2(np.float32(-0.8750387749145276) / (np.float32(1) + np.exp2(np.float32(-1.4426950408889634) * w))) \
        - np.float32(1) + rotator1(phase)
    return d.astype(np.float32).astype(_H)


def _fp16_state_step(state, neg_kk, bvec, wd, k, v, r):
    """The half2 recurrence of both kernels (native_wkv_fp16.py:279-300, 398-425) for state [...,64(i),64(j)] fp16 and
    per-channel fp16 vectors [...,64]: returns (new_state, recurrent [...,64(i)])."""
    st = np.asarray(state, _H).copy()
    lead = st.shape[:-2]
    sa2 = np.zeros(lead + (64, 2), _H)                       # half2 accumulator per row i: lanes = even / odd columns
    for j in range(32):
        sa2 = _hfma(neg_kk[..., None, 2 * j:2 * j + 2], st[..., :, 2 * j:2 * j + 2], sa2)
    sa = _hadd(sa2[..., 0], sa2[..., 1])                     # [...,64(i)]
    y2 = np.zeros(lead + (64, 2), _H)
    vi = np.asarray(v, _H)[..., :, None]
    for j in range(32):
        sl = slice(2 * j, 2 * j + 2)
        s = st[..., :, sl]
        s = _hfma(s, wd[..., None, sl], _hfma(k[..., None, sl], vi, _hfma(sa[..., None], bvec[..., None, sl], s)))
        st[..., :, sl] = s
        y2 = _hfma(s, r[..., None, sl], y2)
    return st, _hadd(y2[..., 0], y2[..., 1])


def native_fp16_recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, state, g, k_k, k_a, r_k, gn_w, gn_b, elapsed, eps):
    """native_wkv_fp16.py:200-333.  Vectors [B,H,64] fp16, state [B,H,64,64] fp16, per-head parameters [H,64] /
    [H*64], elapsed [B] int.  Returns (prepared [B,H,64] fp16, new_state fp16)."""
    B, H, N = np.asarray(r).shape
    f = lambda x: np.asarray(x, _H).astype(np.float32)
    par = lambda x: np.asarray(x, _H).reshape(H, N).astype(np.float32)[None]
    kk_un = f(k_raw) * par(k_k)
    nrm = np.sqrt((kk_un * kk_un).sum(-1, keepdims=True, dtype=np.float32))
    kk_val = kk_un / np.maximum(nrm, np.float32(1e-12))
    af, ka = f(a), par(k_a)
    k_val = (f(k_raw) * (af * ka + (np.float32(1) - ka))).astype(_H)
    kk_h = kk_val.astype(_H)
    bvec = (kk_h.astype(np.float32) * af).astype(_H)
    phase = np.asarray(elapsed, np.int64).reshape(B, 1, 1) + (np.arange(H).reshape(1, H, 1) * N + np.arange(N).reshape(1, 1, N))
    wd = w_delta(w_raw, phase)
    new_state, rec = _fp16_state_step(state, -kk_h, bvec, wd, k_val, np.asarray(v, _H), np.asarray(r, _H))
    rec = rec.astype(np.float32)
    mean = rec.mean(-1, keepdims=True, dtype=np.float32)
    cen = rec - mean
    var = (cen * cen).mean(-1, keepdims=True, dtype=np.float32)
    corr = (f(r) * k_val.astype(np.float32) * par(r_k)).sum(-1, keepdims=True, dtype=np.float32)
    prepared = (cen / np.sqrt(var + np.float32(eps)) * par(gn_w) + par(gn_b) + corr * f(v)) * f(g)
    return prepared.astype(_H), new_state


def native_fp16_sequence(r, w, k, v, neg_kk, kka, state, elapsed, w0=None):
    """native_wkv_fp16.py:335-452: [B,T,H,64] fp16 operands, state [B,H,64,64] fp16.  Token t uses the dither phase
    elapsed[b] + h*64 + j + t.  Returns (y [B,T,H,64] fp16, final_state fp16)."""
    B, T, H, N = np.asarray(r).shape
    st = np.asarray(state, _H).copy()
    y = np.zeros((B, T, H, N), _H)
    base = np.asarray(elapsed, np.int64).reshape(B, 1, 1) + (np.arange(H).reshape(1, H, 1) * N + np.arange(N).reshape(1, 1, N))
    w0v = None if w0 is None else np.asarray(w0, _H).reshape(1, H, N)
    for t in range(T):
        wd = w_delta(np.asarray(w, _H)[:, t], base + t, w0v)
        st, y[:, t] = _fp16_state_step(st, np.asarray(neg_kk, _H)[:, t], np.asarray(kka, _H)[:, t], wd,
                                       np.asarray(k, _H)[:, t], np.asarray(v, _H)[:, t], np.asarray(r, _H)[:, t])
    return y, st
