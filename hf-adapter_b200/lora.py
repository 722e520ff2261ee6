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


def small_gemm_group(xs, weights, biases=None, acts=None, outs=None):
    """One launch for up to four independent small linears ``out_i = act_i(x_i @ W_i.T + b_i)`` sharing the row
    count (fp16/bf16: tensor-core kernel, 64-row blocks; fp32: one ``dense_small`` call per problem)."""
    n = len(xs)
    biases = list(biases) if biases is not None else [None] * n
    acts = list(acts) if acts is not None else [0] * n
    x2 = [x.reshape(-1, int(x.shape[-1])).contiguous() for x in xs]
    M = int(x2[0].shape[0])
    ws = [w.contiguous() for w in weights]
    for x, w in zip(x2, ws):
        if int(x.shape[0]) != M:
            raise ValueError("all problems must have the same number of rows")
        if w.dim() != 2 or int(w.shape[1]) != int(x.shape[1]):
            raise ValueError(f"weight must be [out, {int(x.shape[1])}], got {tuple(w.shape)}")
    if M > 16384 or x2[0].dtype == torch.float32 or n > 4 or any(int(w.shape[1]) % 8 for w in ws):
        res = [dense_small(x, w, b, act_out=a) for x, w, b, a in zip(xs, ws, biases, acts)]
        if outs is not None:
            for o, r in zip(outs, res):
                o.copy_(r.reshape(o.shape))
            return list(outs)
        return res
    bs = [None if b is None else b.contiguous() for b in biases]
    require_cuda(*x2, *ws, *bs, what="small_gemm_group")
    same_dtype(x2[0], *x2, *ws, *bs, what="small_gemm_group")
    if outs is None:
        outs = [torch.empty((M, int(w.shape[0])), device=x.device, dtype=x.dtype) for x, w in zip(x2, ws)]
    xp, _k1 = _lib.ptr_array([t.data_ptr() for t in x2])
    wp, _k2 = _lib.ptr_array([t.data_ptr() for t in ws])
    bp, _k3 = _lib.ptr_array([0 if t is None else t.data_ptr() for t in bs])
    op, _k4 = _lib.ptr_array([t.data_ptr() for t in outs])
    IA = _lib.c_int * n
    _lib.check(_lib.lib.rwkv7_small_gemm_group(n, xp, wp, bp, op, IA(*[int(w.shape[1]) for w in ws]),
                                               IA(*[int(w.shape[0]) for w in ws]), IA(*acts), M, dt_code(x2[0]),
                                               stream_ptr(x2[0])), "small_gemm_group")
    return [o.reshape(*x.shape[:-1], int(w.shape[0])) for o, x, w in zip(outs, xs, ws)]


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
    hw, ha = small_gemm_group((xw, xa), (w_down_weight, a_down_weight), acts=(_TANH, _NONE))
    w, a = small_gemm_group((hw, ha), (w_up_weight, a_up_weight), (w_up_bias, a_up_bias))
    return w, a


def fused_wag_lora(xw, xa, xg, w_down_weight, a_down_weight, g_down_weight, w_up_weight, a_up_weight, g_up_weight,
                   w_up_bias=None, a_up_bias=None, g_up_bias=None, *, block_m: int = 64, block_r: int = 64,
                   block_k: int = 64, force_fallback: bool = False):
    no_fallback(force_fallback, "fused_wag_lora")
    _check_pair(xw, w_down_weight, w_up_weight, w_up_bias, "w")
    _check_pair(xa, a_down_weight, a_up_weight, a_up_bias, "a")
    _check_pair(xg, g_down_weight, g_up_weight, g_up_bias, "g")
    hs = small_gemm_group((xw, xa, xg), (w_down_weight, a_down_weight, g_down_weight), acts=(_TANH, _NONE, _SIGMOID))
    w, a, g = small_gemm_group(hs, (w_up_weight, a_up_weight, g_up_weight), (w_up_bias, a_up_bias, g_up_bias))
    return w, a, g


def fused_wavg_lora(xw, xa, xg, xv, w_down_weight, a_down_weight, g_down_weight, v_down_weight, w_up_weight,
                    a_up_weight, g_up_weight, v_up_weight, w_up_bias=None, a_up_bias=None, g_up_bias=None,
                    v_up_bias=None, *, block_m: int = 64, block_r: int = 64, block_k: int = 64, num_warps: int = 4,
                    force_fallback: bool = False):
    """Two launches (all downs, all ups).  Returns raw ``w``, PRE-sigmoid ``a``, ``g`` and POST-sigmoid ``v_gate``."""
    no_fallback(force_fallback, "fused_wavg_lora")
    _check_pair(xw, w_down_weight, w_up_weight, w_up_bias, "w")
    _check_pair(xa, a_down_weight, a_up_weight, a_up_bias, "a")
    _check_pair(xg, g_down_weight, g_up_weight, g_up_bias, "g")
    _check_pair(xv, v_down_weight, v_up_weight, v_up_bias, "v")
    hs = small_gemm_group((xw, xa, xg, xv), (w_down_weight, a_down_weight, g_down_weight, v_down_weight),
                          acts=(_TANH, _NONE, _SIGMOID, _NONE))
    w, a, g, v_gate = small_gemm_group(hs, (w_up_weight, a_up_weight, g_up_weight, v_up_weight),
                                       (w_up_bias, a_up_bias, g_up_bias, v_up_bias), acts=(_NONE, _NONE, _NONE, _SIGMOID))
    return w, a, g, v_gate
