"""Grouped LoRA operators with the reference's signatures (rwkv7_hf/fused_lora.py:409,559,706):
``w = up(tanh(down(xw))) + b``, ``a = up(down(xa)) + b`` (pre-sigmoid), ``g = up(sigmoid(down(xg)))``,
``v_gate = sigmoid(up(down(xv)) + b)``.  Weights are ``nn.Linear`` style ``[out, in]``."""
from __future__ import annotations

import torch

from . import _lib
from ._util import dt_code, no_fallback, ptr, require_cuda, same_dtype, stream_ptr

_NONE, _TANH, _SIGMOID = 0, 1, 2


def dense_small(x, weight, bias=None, *, act_in: int = 0, act_out: int = 0, out=None):
    """out = act_out(act_in(x) @ weight.T + bias) on the CUDA-core small-linear kernel."""
    K = int(x.shape[-1])
    x2 = x.reshape(-1, K).contiguous()
    if weight.dim() != 2 or int(weight.shape[1]) != K:
        raise ValueError(f"weight must be [out, {K}], got {tuple(weight.shape)}")
    Nout = int(weight.shape[0])
    w = weight.contiguous()
    b = None if bias is None else bias.contiguous()
    require_cuda(x2, w, b, what="dense_small")
    same_dtype(x2, w, b, what="dense_small")
    if out is None:
        out = torch.empty((x2.shape[0], Nout), device=x2.device, dtype=x2.dtype)
    _lib.check(_lib.lib.rwkv7_dense_small(ptr(x2), ptr(w), ptr(b), ptr(out), int(x2.shape[0]), K, Nout, act_in,
                                          act_out, dt_code(x2), stream_ptr(x2)), "dense_small")
    return out.reshape(*x.shape[:-1], Nout)


def _check_pair(x, down, up, bias, name):
    hidden = int(x.shape[-1])
    if down.dim() != 2 or int(down.shape[1]) != hidden:
        raise ValueError(f"{name}_down_weight must be [rank, {hidden}], got {tuple(down.shape)}")
    if up.dim() != 2 or int(up.shape[1]) != int(down.shape[0]):
        raise ValueError(f"{name}_up_weight must be [out, {int(down.shape[0])}], got {tuple(up.shape)}")
    if bias is not None and int(bias.numel()) != int(up.shape[0]):
        raise ValueError(f"{name}_up_bias must contain {int(up.shape[0])} values")


def fused_wa_lora(xw, xa, w_down_weight, a_down_weight, w_up_weight, a_up_weight, w_up_bias=None, a_up_bias=None, *,
                  block_m: int = 64, block_r: int = 64, block_k: int = 64, force_fallback: bool = False):
    no_fallback(force_fallback, "fused_wa_lora")
    _check_pair(xw, w_down_weight, w_up_weight, w_up_bias, "w")
    _check_pair(xa, a_down_weight, a_up_weight, a_up_bias, "a")
    w = dense_small(dense_small(xw, w_down_weight, act_out=_TANH), w_up_weight, w_up_bias)
    a = dense_small(dense_small(xa, a_down_weight), a_up_weight, a_up_bias)
    return w, a


def fused_wag_lora(xw, xa, xg, w_down_weight, a_down_weight, g_down_weight, w_up_weight, a_up_weight, g_up_weight,
                   w_up_bias=None, a_up_bias=None, g_up_bias=None, *, block_m: int = 64, block_r: int = 64,
                   block_k: int = 64, force_fallback: bool = False):
    no_fallback(force_fallback, "fused_wag_lora")
    w, a = fused_wa_lora(xw, xa, w_down_weight, a_down_weight, w_up_weight, a_up_weight, w_up_bias, a_up_bias)
    _check_pair(xg, g_down_weight, g_up_weight, g_up_bias, "g")
    g = dense_small(dense_small(xg, g_down_weight, act_out=_SIGMOID), g_up_weight, g_up_bias)
    return w, a, g


def fused_wavg_lora(xw, xa, xg, xv, w_down_weight, a_down_weight, g_down_weight, v_down_weight, w_up_weight,
                    a_up_weight, g_up_weight, v_up_weight, w_up_bias=None, a_up_bias=None, g_up_bias=None,
                    v_up_bias=None, *, block_m: int = 64, block_r: int = 64, block_k: int = 64, num_warps: int = 4,
                    force_fallback: bool = False):
    """Returns raw ``w``, PRE-sigmoid ``a``, ``g`` and POST-sigmoid ``v_gate``."""
    no_fallback(force_fallback, "fused_wavg_lora")
    w, a, g = fused_wag_lora(xw, xa, xg, w_down_weight, a_down_weight, g_down_weight, w_up_weight, a_up_weight,
                             g_up_weight, w_up_bias, a_up_bias, g_up_bias)
    _check_pair(xv, v_down_weight, v_up_weight, v_up_bias, "v")
    v_gate = dense_small(dense_small(xv, v_down_weight), v_up_weight, v_up_bias, act_out=_SIGMOID)
    return w, a, g, v_gate
