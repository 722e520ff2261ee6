"""LayerNorm + token-shift mixing operators with the reference's signatures
(rwkv7_hf/fused_decode_norm_mix.py:161,296 and rwkv7_hf/fused_time_mix.py:340,413,470)."""
from __future__ import annotations

import torch

from . import _lib
from ._util import dt_code, no_fallback, ptr, require_cuda, same_dtype, stream_ptr


def _rows(x, name):
    if x.dim() == 1:
        return x.reshape(1, -1), tuple(x.shape)
    if x.dim() == 2:
        return x, tuple(x.shape)
    raise ValueError(f"{name} must be [hidden] or [batch, hidden], got {tuple(x.shape)}")


def _vec(value, hidden, name):
    if value is None or int(value.numel()) != hidden:
        shape = None if value is None else tuple(value.shape)
        raise ValueError(f"{name} must contain hidden={hidden} values; got {shape}")
    return value.reshape(hidden).contiguous()


def _check_slots(slot_ids, rows, pool, hidden):
    if not (slot_ids.is_cuda and slot_ids.dtype == torch.int32 and slot_ids.is_contiguous() and int(slot_ids.numel()) == rows):
        raise ValueError("slot_ids must be a contiguous CUDA int32 tensor with one entry per row")
    if pool.dim() != 2 or int(pool.shape[1]) != hidden:
        raise ValueError(f"with slot_ids, previous must be a pool [capacity, {hidden}]")


def fused_attn_norm_mix6_decode(x, previous, norm_weight, norm_bias, mix_r, mix_w, mix_k, mix_v, mix_a, mix_g, *,
                                eps: float = 1e-5, num_warps: int = 4, stack_rkv: bool = False,
                                stack_wav: bool = False, stack_rkv_wagv: bool = False, force_fallback: bool = False,
                                slot_ids=None):
    """Layer-normalise ``x``, update ``previous`` in place, and emit the six time mixes (r,w,k,v,a,g).
    The ``stack_*`` options place outputs in one allocation in the same slot orders as the reference.
    ``slot_ids`` (int32 ``[rows]``, an extension): ``previous`` is a state pool ``[capacity, D]`` and row ``b`` of ``x``
    uses its row ``slot_ids[b]``."""
    no_fallback(force_fallback, "fused_attn_norm_mix6_decode")
    x2, shape = _rows(x, "x")
    prev2, prev_shape = _rows(previous, "previous")
    if slot_ids is not None:
        _check_slots(slot_ids, int(x2.shape[0]), prev2, int(x2.shape[1]))
    elif prev_shape != shape:
        raise ValueError("x and previous must have identical shapes")
    hidden = int(x2.shape[1])
    names = ("norm_weight", "norm_bias", "mix_r", "mix_w", "mix_k", "mix_v", "mix_a", "mix_g")
    params = [_vec(v, hidden, n) for v, n in zip((norm_weight, norm_bias, mix_r, mix_w, mix_k, mix_v, mix_a, mix_g), names)]
    require_cuda(x2, prev2, *params, what="fused_attn_norm_mix6_decode")
    same_dtype(x2, prev2, *params, what="fused_attn_norm_mix6_decode")
    if not prev2.is_contiguous():
        raise ValueError("previous must be contiguous (it is updated in place)")
    x_c = x2.contiguous()
    if x_c.data_ptr() == prev2.data_ptr():
        raise ValueError("x and previous must not alias")
    rows = int(x_c.shape[0])
    new = lambda n: torch.empty((n, rows, hidden), device=x_c.device, dtype=x_c.dtype)
    if stack_rkv_wagv:
        s = new(6)  # physical order R,K,V,W,A,G
        outs = (s[0], s[3], s[1], s[2], s[4], s[5])
    elif stack_rkv:
        s, o = new(3), new(3)
        outs = (s[0], o[0], s[1], s[2], o[1], o[2])
    elif stack_wav:
        s, o = new(3), new(3)  # physical order W,A,V
        outs = (o[0], s[0], o[1], s[2], s[1], o[2])
    else:
        s = new(6)
        outs = tuple(s[i] for i in range(6))
    mixes_p, _k1 = _lib.ptr_array([p.data_ptr() for p in params[2:]])
    outs_p, _k2 = _lib.ptr_array([o.data_ptr() for o in outs])
    if slot_ids is not None:
        _lib.check(_lib.lib.rwkv7_attn_norm_mix6_pool(ptr(x_c), ptr(prev2), ptr(slot_ids), ptr(params[0]), ptr(params[1]),
                                                      mixes_p, outs_p, rows, hidden, float(eps), dt_code(x_c),
                                                      stream_ptr(x_c)), "fused_attn_norm_mix6_decode")
    else:
        _lib.check(_lib.lib.rwkv7_attn_norm_mix6(ptr(x_c), ptr(prev2), ptr(params[0]), ptr(params[1]), mixes_p, outs_p,
                                                 rows, hidden, float(eps), dt_code(x_c), stream_ptr(x_c)),
                   "fused_attn_norm_mix6_decode")
    return tuple(o.reshape(shape) for o in outs)


def fused_ffn_add_norm_mix_decode(residual, attn_out, previous, norm_weight, norm_bias, mix, *, eps: float = 1e-5,
                                  num_warps: int = 4, force_fallback: bool = False, slot_ids=None):
    """x = residual + attn_out; h = LN(x); mixed = h + (previous - h) * mix; previous <- h.
    Returns ``(x, mixed)``.  ``slot_ids``: as in ``fused_attn_norm_mix6_decode``."""
    no_fallback(force_fallback, "fused_ffn_add_norm_mix_decode")
    res2, shape = _rows(residual, "residual")
    attn2, attn_shape = _rows(attn_out, "attn_out")
    prev2, prev_shape = _rows(previous, "previous")
    if slot_ids is not None:
        _check_slots(slot_ids, int(res2.shape[0]), prev2, int(res2.shape[1]))
        prev_shape = shape
    if attn_shape != shape or prev_shape != shape:
        raise ValueError("residual, attn_out, and previous must have identical shapes")
    hidden = int(res2.shape[1])
    w, b, m = (_vec(v, hidden, n) for v, n in ((norm_weight, "norm_weight"), (norm_bias, "norm_bias"), (mix, "mix")))
    require_cuda(res2, attn2, prev2, w, b, m, what="fused_ffn_add_norm_mix_decode")
    same_dtype(res2, attn2, prev2, w, b, m, what="fused_ffn_add_norm_mix_decode")
    if not prev2.is_contiguous():
        raise ValueError("previous must be contiguous (it is updated in place)")
    res_c, attn_c = res2.contiguous(), attn2.contiguous()
    res_out, mixed = torch.empty_like(res_c), torch.empty_like(res_c)
    if slot_ids is not None:
        _lib.check(_lib.lib.rwkv7_ffn_add_norm_mix_pool(ptr(res_c), ptr(attn_c), ptr(prev2), ptr(slot_ids), ptr(w), ptr(b),
                                                        ptr(m), ptr(res_out), ptr(mixed), int(res_c.shape[0]), hidden,
                                                        float(eps), dt_code(res_c), stream_ptr(res_c)),
                   "fused_ffn_add_norm_mix_decode")
    else:
        _lib.check(_lib.lib.rwkv7_ffn_add_norm_mix(ptr(res_c), ptr(attn_c), ptr(prev2), ptr(w), ptr(b), ptr(m),
                                                   ptr(res_out), ptr(mixed), int(res_c.shape[0]), hidden, float(eps),
                                                   dt_code(res_c), stream_ptr(res_c)), "fused_ffn_add_norm_mix_decode")
    return res_out.reshape(shape), mixed.reshape(shape)


def layer_norm(x, weight, bias, eps: float = 1e-5, out=None):
    """Plain LayerNorm over the last axis (layer-0 pre_norm and the final norm)."""
    hidden = int(x.shape[-1])
    x2 = x.reshape(-1, hidden).contiguous()
    require_cuda(x2, weight, bias, what="layer_norm")
    same_dtype(x2, weight, bias, what="layer_norm")
    if out is None:
        out = torch.empty_like(x2)
    _lib.check(_lib.lib.rwkv7_layer_norm(ptr(x2), ptr(weight.contiguous()), ptr(bias.contiguous()), ptr(out),
                                         int(x2.shape[0]), hidden, float(eps), dt_code(x2), stream_ptr(x2)), "layer_norm")
    return out.reshape(x.shape)


def _seq_mix(x, initial_prev, mixes, workspace, name, strict=False):
    if x.dim() != 3:
        raise ValueError(f"{name}: x must be [batch, tokens, hidden]")
    B, T, D = (int(v) for v in x.shape)
    initial = initial_prev.reshape(B, D).contiguous()
    flat = [_vec(m, D, "mix") for m in mixes]
    require_cuda(x, initial, *flat, what=name)
    same_dtype(x, initial, *flat, what=name)
    src = x.contiguous()
    if strict and x.dtype != torch.float16:
        strict = False  # the reference applies strict rounding to fp16 sources only (fused_time_mix.py:448,509)
    n = len(flat)
    expected = (n, B, T, D) if name == "fused_attn_sequence_shift_mix" else (B, T, D)
    if workspace is not None and tuple(workspace.shape) == expected and workspace.device == x.device \
            and workspace.dtype == x.dtype and workspace.is_contiguous():
        storage = workspace
    else:
        storage = torch.empty(expected, device=x.device, dtype=x.dtype)
    nxt = torch.empty((B, D), device=x.device, dtype=x.dtype)
    return src, initial, flat, storage, nxt, (B, T, D), int(bool(strict))


def fused_attn_sequence_shift_mix(x, initial_prev, *mixes, block_size: int = 256, num_warps: int = 4, workspace=None,
                                  strict_fp16_rounding: bool = False):
    """Shift-mix a whole ``[B,T,C]`` sequence.  Returns ``(xr,xw,xk,xv,xa,xg,next_state)``; the six
    streams share one ``[6,B,T,C]`` allocation in the physical order R,K,V,W,A,G like the reference.
    ``strict_fp16_rounding=True`` (fp16 sources) rounds the difference, the product and the sum separately, as the
    reference's strict lowering and eager PyTorch do (rwkv7_hf/fused_time_mix.py:63-134)."""
    if len(mixes) != 6:
        raise ValueError("fused_attn_sequence_shift_mix requires six mix vectors")
    src, initial, flat, storage, nxt, (B, T, D), strict = _seq_mix(x, initial_prev, mixes, workspace,
                                                                    "fused_attn_sequence_shift_mix", strict_fp16_rounding)
    slots = storage.unbind(0)
    outs = (slots[0], slots[3], slots[1], slots[2], slots[4], slots[5])
    mp, _k1 = _lib.ptr_array([m.data_ptr() for m in flat])
    op, _k2 = _lib.ptr_array([o.data_ptr() for o in outs])
    _lib.check(_lib.lib.rwkv7_seq_shift_mix(ptr(src), ptr(initial), mp, op, ptr(nxt), B, T, D, 6, strict, dt_code(src),
                                            stream_ptr(src)), "fused_attn_sequence_shift_mix")
    return (*outs, nxt)


def fused_ffn_sequence_shift_mix(x, initial_prev, mix, block_size: int = 256, num_warps: int = 4, workspace=None,
                                 strict_fp16_rounding: bool = False):
    """Single-stream sequence shift-mix for the FFN (rwkv7_hf/fused_time_mix.py:470; all parameters positional or
    keyword as there; ``workspace`` is a ``[B,T,C]`` output buffer).  Returns ``(mixed, next_state)``."""
    src, initial, flat, storage, nxt, (B, T, D), strict = _seq_mix(x, initial_prev, (mix,), workspace,
                                                                    "fused_ffn_sequence_shift_mix", strict_fp16_rounding)
    mp, _k1 = _lib.ptr_array([flat[0].data_ptr()])
    op, _k2 = _lib.ptr_array([storage.data_ptr()])
    _lib.check(_lib.lib.rwkv7_seq_shift_mix(ptr(src), ptr(initial), mp, op, ptr(nxt), B, T, D, 1, strict, dt_code(src),
                                            stream_ptr(src)), "fused_ffn_sequence_shift_mix")
    return storage, nxt


def fused_attn_shift_mix(x, prev, x_r, x_w, x_k, x_v, x_a, x_g, *, block_size: int = 256, force_fallback: bool = False):
    """Six mixes of ``x`` against an explicit previous tensor of the same shape, ``[batch, hidden]`` or
    ``[batch, tokens, hidden]`` (rwkv7_hf/fused_time_mix.py:340): each row is a one-token sequence whose initial state
    is its row of ``prev``.  Mix vectors may have any shape with ``hidden`` elements."""
    no_fallback(force_fallback, "fused_attn_shift_mix")
    if x.shape != prev.shape:
        raise ValueError("x and prev must have identical flattened shapes")
    D = int(x.shape[-1])
    x3 = x.reshape(-1, 1, D)
    outs = fused_attn_sequence_shift_mix(x3, prev.reshape(-1, D), *(m.reshape(-1) for m in (x_r, x_w, x_k, x_v, x_a, x_g)))
    return tuple(o.reshape(x.shape) for o in outs[:6])
