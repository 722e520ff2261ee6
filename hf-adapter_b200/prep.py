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


def fused_prefill_kv_kk_prep(k_raw, v_raw, a, k_k, k_a, *, v_first=None, v_gate=None, num_heads: int, head_dim: int,
                             force_fallback: bool = False, a_is_raw: bool = False, v_gate_is_raw: bool = False):
    """State prep without the decay (rwkv7_hf/fused_prefill.py:324), the companion of the raw-w scan.
    Returns ``(k_adjusted, v_interpolated, kk_normalized)`` in the input layout.  ``a_is_raw`` / ``v_gate_is_raw``
    (extensions, as in ``fused_prefill_state_prep``): the sigmoid of ``a`` / of the v gate is applied in the kernel."""
    no_fallback(force_fallback, "fused_prefill_kv_kk_prep")
    hidden = int(num_heads) * int(head_dim)
    k2, prefix = _flat(k_raw, hidden, "k_raw")
    v2, vp = _flat(v_raw, hidden, "v_raw")
    a2, ap = _flat(a, hidden, "a")
    if vp != prefix or ap != prefix:
        raise ValueError("k_raw, v_raw and a must have identical layouts")
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
    require_cuda(k2, v2, a2, kk_c, ka_c, vf2, vg2, what="fused_prefill_kv_kk_prep")
    same_dtype(k2, v2, a2, kk_c, ka_c, vf2, vg2, what="fused_prefill_kv_kk_prep")
    rows = int(k2.shape[0])
    k_out, v_out, kk_out = torch.empty_like(k2), torch.empty_like(k2), torch.empty_like(k2)
    _lib.check(_lib.lib.rwkv7_prefill_state_prep(
        None, ptr(k2), ptr(v2), ptr(a2), ptr(kk_c), ptr(ka_c), ptr(vf2), ptr(vg2), None, ptr(k_out), ptr(v_out),
        ptr(kk_out), rows, int(num_heads), int(head_dim), int(bool(a_is_raw)), int(bool(v_gate_is_raw)), 0, dt_code(k2),
        stream_ptr(k2)), "fused_prefill_kv_kk_prep")
    rs = lambda t: t.reshape(*prefix, hidden)
    return rs(k_out), rs(v_out), rs(kk_out)


def fused_attn_output_project(recurrent_out, r, k, v, g, r_k, group_norm_weight, group_norm_bias, o_proj_weight,
                              o_proj_bias=None, *, num_heads: int, head_dim: int, head_v_dim: int, eps: float,
                              block_m: int = 32, force_fallback: bool = False):
    """Output prep followed by ``o_proj`` (rwkv7_hf/fused_output.py:278): the prep kernel, then this library's GEMM (bias in
    its epilogue; a quantised ``o_proj`` module is applied as a callable)."""
    no_fallback(force_fallback, "fused_attn_output_project")
    prepared = fused_attn_output_prepare(recurrent_out, r, k, v, g, r_k, group_norm_weight, group_norm_bias,
                                         num_heads=num_heads, head_dim=head_dim, head_v_dim=head_v_dim, eps=eps)
    if callable(o_proj_weight) and not isinstance(o_proj_weight, torch.Tensor):
        y = o_proj_weight(prepared)
        return y if o_proj_bias is None else y + o_proj_bias
    value_dim = int(num_heads) * int(head_v_dim)
    if o_proj_weight.dim() != 2 or int(o_proj_weight.shape[1]) != value_dim:
        raise ValueError(f"o_proj_weight must be [output_dim, {value_dim}], got {tuple(o_proj_weight.shape)}")
    if o_proj_bias is not None and (o_proj_bias.dim() != 1 or int(o_proj_bias.shape[0]) != int(o_proj_weight.shape[0])):
        raise ValueError(f"o_proj_bias must be [{int(o_proj_weight.shape[0])}]")
    from . import gemm as _gemm
    if _gemm.takes(prepared, o_proj_weight) and (o_proj_bias is None or o_proj_bias.dtype == prepared.dtype):
        return _gemm.dense_linear(prepared, o_proj_weight, o_proj_bias)
    return torch.nn.functional.linear(prepared, o_proj_weight, o_proj_bias)


def _dense(x, weight, *, relu2: bool = False):
    """A dense projection: this library's GEMM with the relu^2 fused for fp16 / bf16, a library GEMM plus the relu^2
    kernel for fp32 operands (the tensor-core kernel has no fp32-operand form)."""
    from . import gemm as _gemm
    if _gemm.takes(x, weight):
        return _gemm.dense_linear(x, weight, relu2=relu2)
    y = torch.nn.functional.linear(x, weight)
    return relu2_(y) if relu2 else y


def relu2_(x):
    """In place ``max(x, 0)**2``."""
    require_cuda(x, what="relu2")
    if not x.is_contiguous() or int(x.numel()) % 8:
        raise ValueError("relu2 needs a contiguous tensor whose element count is a multiple of 8")
    _lib.check(_lib.lib.rwkv7_relu2(ptr(x), ptr(x), int(x.numel()), dt_code(x), stream_ptr(x)), "relu2")
    return x


def _ffn_checks(hidden, mix_x, key_weight, value_weight):
    mix = mix_x.reshape(-1)
    if int(mix.shape[0]) != hidden:
        raise ValueError(f"mix_x must have {hidden} elements, got {int(mix.shape[0])}")
    if key_weight.dim() != 2 or int(key_weight.shape[1]) != hidden:
        raise ValueError(f"key_weight must be [intermediate, {hidden}], got {tuple(key_weight.shape)}")
    inter = int(key_weight.shape[0])
    if value_weight.dim() != 2 or tuple(value_weight.shape) != (hidden, inter):
        raise ValueError(f"value_weight must be [{hidden}, {inter}], got {tuple(value_weight.shape)}")
    return mix.contiguous()


def fused_ffn(hidden_states, prev_states, mix_x, key_weight, value_weight, *, block_m: int = 64, block_k: int = 64,
              force_fallback: bool = False):
    """One-token FFN with dense weights (rwkv7_hf/fused_ffn.py:394): shift-mix kernel, key GEMM, relu^2 kernel,
    value GEMM.  Returns ``(out, next_state)``; ``next_state`` is the input."""
    from . import norm_mix as _nm
    no_fallback(force_fallback, "fused_ffn")
    had_seq = hidden_states.dim() == 3
    if had_seq and int(hidden_states.shape[1]) != 1:
        raise ValueError(f"hidden_states must be [batch, 1, hidden] or [batch, hidden], got {tuple(hidden_states.shape)}")
    hidden = int(hidden_states.shape[-1])
    x2 = hidden_states.reshape(-1, hidden)
    prev2 = prev_states.reshape(-1, hidden)
    if tuple(prev2.shape) != tuple(x2.shape):
        raise ValueError("hidden_states and prev_states must have identical flattened shape/layout")
    mix = _ffn_checks(hidden, mix_x, key_weight, value_weight)
    mixed, _ = _nm.fused_ffn_sequence_shift_mix(x2.reshape(-1, 1, hidden), prev2.contiguous(), mix)
    mid = _dense(mixed.reshape(-1, hidden), key_weight, relu2=True)
    out = _dense(mid, value_weight)
    if had_seq:
        return out.unsqueeze(1), hidden_states[:, -1:].contiguous()
    return out, hidden_states.contiguous()


def fused_sequence_ffn(hidden_states, prev_states, mix_x, key_weight, value_weight, *, block_m: int = 128,
                       block_n: int = 128, key_block_k: int = 32, value_block_k: int = 64, group_m: int = 8,
                       num_stages: int = 3, num_warps: int = 4, workspace=None, force_fallback: bool = False):
    """Sequence FFN (rwkv7_hf/fused_ffn.py:245): ``[B,T,H]`` in, ``([B,T,H], next_state [B,H])`` out."""
    from . import norm_mix as _nm
    no_fallback(force_fallback, "fused_sequence_ffn")
    if int(num_warps) not in {1, 2, 4, 8}:
        raise ValueError("num_warps must be one of 1, 2, 4, or 8")
    if int(num_stages) not in {1, 2, 3, 4, 5}:
        raise ValueError("num_stages must be between 1 and 5")
    if hidden_states.dim() != 3:
        raise ValueError(f"hidden_states must be [B,T,H], got {tuple(hidden_states.shape)}")
    batch, tokens, hidden = (int(v) for v in hidden_states.shape)
    if prev_states.dim() == 3 and int(prev_states.shape[1]) == 1:
        prev_states = prev_states[:, 0, :]
    if prev_states.dim() != 2 or tuple(prev_states.shape) != (batch, hidden):
        raise ValueError(f"prev_states must be [{batch},{hidden}], got {tuple(prev_states.shape)}")
    mix = _ffn_checks(hidden, mix_x, key_weight, value_weight)
    mixed, nxt = _nm.fused_ffn_sequence_shift_mix(hidden_states, prev_states.contiguous(), mix)
    mid = _dense(mixed.reshape(batch * tokens, hidden), key_weight, relu2=True)
    out = _dense(mid, value_weight)
    return out.reshape(batch, tokens, hidden), nxt
