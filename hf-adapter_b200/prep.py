"""Prefill state preparation and attention-output preparation with the reference's signatures
(rwkv7_hf/fused_prefill.py:184,324 and rwkv7_hf/fused_output.py:190)."""
from __future__ import annotations

import torch

from . import _lib
from ._util import dt_code, no_fallback, ptr, require_cuda, same_dtype, stream_ptr


def _flat(x, hidden, name):
    if int(x.shape[-1]) != hidden:
        raise ValueError(f"{name} must end in hidden={hidden}; got {tuple(x.shape)}")
    return x.reshape(-1, hidden).contiguous(), tuple(x.shape[:-1])


def fused_prefill_state_prep(w_raw, k_raw, v_raw, a, k_k, k_a, *, v_first=None, v_gate=None, num_heads: int,
                             head_dim: int, w_out_dtype: str = "fp32", w_transform: str = "decay",
                             a_is_raw: bool = False, v_gate_is_raw: bool = False, force_fallback: bool = False):
    """Returns ``(w_decay, k_adjusted, v_interpolated, kk_normalized)`` in the input layout."""
    no_fallback(force_fallback, "fused_prefill_state_prep")
    if w_out_dtype not in {"fp32", "input"}:
        raise ValueError(f"w_out_dtype must be 'fp32' or 'input'; got {w_out_dtype!r}")
    if w_transform not in {"decay", "log_decay"}:
        raise ValueError(f"w_transform must be 'decay' or 'log_decay'; got {w_transform!r}")
    hidden = int(num_heads) * int(head_dim)
    w2, prefix = _flat(w_raw, hidden, "w_raw")
    k2, kp = _flat(k_raw, hidden, "k_raw")
    v2, vp = _flat(v_raw, hidden, "v_raw")
    a2, ap = _flat(a, hidden, "a")
    if kp != prefix or vp != prefix or ap != prefix:
        raise ValueError("w_raw, k_raw, v_raw and a must have identical layouts")
    if int(k_k.numel()) != hidden or int(k_a.numel()) != hidden:
        raise ValueError(f"k_k and k_a must have {hidden} elements")
    has_v = v_first is not None and v_gate is not None
    vf2 = vg2 = None
    if has_v:
        vf2, vfp = _flat(v_first, hidden, "v_first")
        vg2, vgp = _flat(v_gate, hidden, "v_gate")
        if vfp != prefix or vgp != prefix:
            raise ValueError("v_first/v_gate layout must match v_raw")
    kk_c, ka_c = k_k.reshape(hidden).contiguous(), k_a.reshape(hidden).contiguous()
    require_cuda(w2, k2, v2, a2, kk_c, ka_c, vf2, vg2, what="fused_prefill_state_prep")
    same_dtype(w2, k2, v2, a2, kk_c, ka_c, vf2, vg2, what="fused_prefill_state_prep")
    rows = int(w2.shape[0])
    w_out = torch.empty((rows, hidden), device=w2.device, dtype=torch.float32)
    k_out, v_out, kk_out = torch.empty_like(k2), torch.empty_like(k2), torch.empty_like(k2)
    _lib.check(_lib.lib.rwkv7_prefill_state_prep(
        ptr(w2), ptr(k2), ptr(v2), ptr(a2), ptr(kk_c), ptr(ka_c), ptr(vf2), ptr(vg2), ptr(w_out), ptr(k_out),
        ptr(v_out), ptr(kk_out), rows, int(num_heads), int(head_dim), int(bool(a_is_raw)), int(bool(v_gate_is_raw)),
        int(w_transform == "log_decay"), dt_code(w2), stream_ptr(w2)), "fused_prefill_state_prep")
    if w_out_dtype == "input":
        w_out = w_out.to(w2.dtype)
    rs = lambda t: t.reshape(*prefix, hidden)
    return rs(w_out), rs(k_out), rs(v_out), rs(kk_out)


def fused_attn_output_prepare(recurrent_out, r, k, v, g, r_k, group_norm_weight, group_norm_bias, *, num_heads: int,
                              head_dim: int, head_v_dim: int, eps: float, force_fallback: bool = False, out=None):
    """(GroupNorm_H(recurrent_out) + (sum_n r k r_k) v) * g; returns a tensor shaped like ``recurrent_out``."""
    no_fallback(force_fallback, "fused_attn_output_prepare")
    if int(head_v_dim) != int(head_dim):
        raise ValueError("head_v_dim must equal head_dim")
    hidden = int(num_heads) * int(head_dim)
    rec2, _ = _flat(recurrent_out, hidden, "recurrent_out")
    rows = int(rec2.shape[0])
    flat_h = lambda t, n: t.reshape(rows, hidden).contiguous() if int(t.numel()) == rows * hidden else _flat(t, hidden, n)[0]
    r2, k2, v2, g2 = (flat_h(t, n) for t, n in ((r, "r"), (k, "k"), (v, "v"), (g, "g")))
    rk, gw, gb = (t.reshape(hidden).contiguous() for t in (r_k, group_norm_weight, group_norm_bias))
    require_cuda(rec2, r2, k2, v2, g2, rk, gw, gb, what="fused_attn_output_prepare")
    same_dtype(rec2, r2, k2, v2, g2, rk, gw, gb, what="fused_attn_output_prepare")
    if out is None:
        out = torch.empty_like(rec2)
    _lib.check(_lib.lib.rwkv7_attn_output_prepare(ptr(rec2), ptr(r2), ptr(k2), ptr(v2), ptr(g2), ptr(rk), ptr(gw),
                                                  ptr(gb), ptr(out), rows, int(num_heads), int(head_dim), float(eps),
                                                  dt_code(rec2), stream_ptr(rec2)), "fused_attn_output_prepare")
    return out.reshape(recurrent_out.shape)
