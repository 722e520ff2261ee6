"""WKV-7 recurrence operators with the reference's signatures.

Mirrors rwkv7_hf/fused_recurrent_update.py (fused_recurrent_update :1214,
fused_recurrent_output_prepare :967, fused_recurrent_output_prepare_raw :1089,
fused_recurrent_scan :1299, _clampw :1420, _output_prepare :1710),
rwkv7_hf/self_chunk_rwkv7.py:33 and rwkv7_hf/dplr_prefill.py:505: same names,
argument order and meaning, same shape errors.  Vectors are ``[B,H,N]`` or flat
``[B,H*N]`` (``[B,T,H,N]`` / ``[B,T,H*N]`` for scans); the output follows the
rank of ``r``; the input state is left untouched and a new state is returned.
The ``*_inplace`` variants are extra entry points for this package's own decode
runner: they overwrite the state and write into caller-provided outputs.
"""
from __future__ import annotations

import torch

from . import _lib
from ._util import dt_code, no_fallback, ptr, require_cuda, same_dtype, stream_ptr


def _state_shape(state, allow_f16: bool = False):
    if state.dim() != 4:
        raise ValueError("state must be shaped [batch, heads, head_dim, head_dim]")
    B, H, N, N2 = (int(v) for v in state.shape)
    if N != N2:
        raise ValueError("state must be square in the last two dimensions")
    if state.dtype != torch.float32 and not (allow_f16 and state.dtype == torch.float16):
        raise ValueError("state must be float32" + (" or float16" if allow_f16 else
                         " (only the output-prepare operators and the scans take a float16 state)"))
    return B, H, N


def _as_bhn(x, B, H, N, name):
    if x.dim() == 3:
        if tuple(x.shape) != (B, H, N):
            raise ValueError(f"{name} must be shaped [batch,{H},{N}] or [batch,{H * N}]; got {tuple(x.shape)}")
        return x.contiguous(), False
    if x.dim() == 2:
        if tuple(x.shape) != (B, H * N):
            raise ValueError(f"{name} must be shaped [batch,{H},{N}] or [batch,{H * N}]; got {tuple(x.shape)}")
        return x.contiguous(), True
    raise ValueError(f"{name} must be shaped [batch,{H},{N}] or [batch,{H * N}]")


def _as_bthn(x, B, H, N, name):
    if x.dim() == 4:
        if int(x.shape[0]) != B or int(x.shape[2]) != H or int(x.shape[3]) != N:
            raise ValueError(f"{name} must be shaped [batch,tokens,{H},{N}] or [batch,tokens,{H * N}]; got {tuple(x.shape)}")
        return x.contiguous(), False
    if x.dim() == 3:
        if int(x.shape[0]) != B or int(x.shape[2]) != H * N:
            raise ValueError(f"{name} must be shaped [batch,tokens,{H},{N}] or [batch,tokens,{H * N}]; got {tuple(x.shape)}")
        return x.contiguous(), True
    raise ValueError(f"{name} must be shaped [batch,tokens,{H},{N}] or [batch,tokens,{H * N}]")


def _w_flag(w, act_dtype):
    if w.dtype == torch.float32 and act_dtype != torch.float32:
        return 1
    if w.dtype != act_dtype:
        raise ValueError(f"w must be float32 or the activation dtype {act_dtype}; got {w.dtype}")
    return 0


def fused_recurrent_update(r, w, k, v, kk, a, state, *, block_n: int = 64, force_fallback: bool = False, out=None,
                           new_state=None):
    """One-token update.  Returns ``(out, new_state)``."""
    no_fallback(force_fallback, "fused_recurrent_update")
    B, H, N = _state_shape(state)
    r_, flat = _as_bhn(r, B, H, N, "r")
    w_, k_, v_, kk_, a_ = (_as_bhn(t, B, H, N, n)[0] for t, n in ((w, "w"), (k, "k"), (v, "v"), (kk, "kk"), (a, "a")))
    require_cuda(r_, w_, k_, v_, kk_, a_, state, what="fused_recurrent_update")
    same_dtype(r_, k_, v_, kk_, a_, what="fused_recurrent_update")
    state_c = state.contiguous()
    if new_state is None:
        new_state = torch.empty_like(state_c)
    if out is None:
        out = torch.empty_like(r_)
    _lib.check(_lib.lib.rwkv7_wkv7_update(ptr(r_), ptr(w_), ptr(k_), ptr(v_), ptr(kk_), ptr(a_), ptr(state_c),
                                          ptr(new_state), ptr(out), B, H, N, dt_code(r_), _w_flag(w_, r_.dtype),
                                          stream_ptr(r_)), "fused_recurrent_update")
    return (out.reshape(B, H * N) if flat else out.reshape(B, H, N)), new_state


def _check_prep_params(H, N, r_k, gn_w, gn_b):
    if int(r_k.numel()) != H * N:
        raise ValueError(f"r_k must be [{H}, {N}], got {tuple(r_k.shape)}")
    if gn_w.dim() != 1 or int(gn_w.shape[0]) != H * N:
        raise ValueError(f"group_norm_weight must be [{H * N}], got {tuple(gn_w.shape)}")
    if gn_b.dim() != 1 or int(gn_b.shape[0]) != H * N:
        raise ValueError(f"group_norm_bias must be [{H * N}], got {tuple(gn_b.shape)}")


def fused_recurrent_output_prepare(r, w, k, v, kk, a, state, g, r_k, group_norm_weight, group_norm_bias, *, eps: float,
                                   block_n: int = 64, force_fallback: bool = False, out=None, new_state=None):
    """Update + GroupNorm + bonus + gate.  Returns ``(prepared, new_state)``."""
    no_fallback(force_fallback, "fused_recurrent_output_prepare")
    B, H, N = _state_shape(state, allow_f16=True)
    r_, flat = _as_bhn(r, B, H, N, "r")
    w_, k_, v_, kk_, a_, g_ = (_as_bhn(t, B, H, N, n)[0] for t, n in
                               ((w, "w"), (k, "k"), (v, "v"), (kk, "kk"), (a, "a"), (g, "g")))
    _check_prep_params(H, N, r_k, group_norm_weight, group_norm_bias)
    rk_, gw_, gb_ = r_k.contiguous(), group_norm_weight.contiguous(), group_norm_bias.contiguous()
    require_cuda(r_, w_, k_, v_, kk_, a_, g_, state, rk_, gw_, gb_, what="fused_recurrent_output_prepare")
    same_dtype(r_, k_, v_, kk_, a_, g_, rk_, gw_, gb_, what="fused_recurrent_output_prepare")
    state_c = state.contiguous()
    if new_state is None:
        new_state = torch.empty_like(state_c)
    if out is None:
        out = torch.empty_like(r_)
    fn = _lib.lib.rwkv7_wkv7_output_prepare if state_c.dtype == torch.float32 else _lib.lib.rwkv7_wkv7_output_prepare_f16state
    _lib.check(fn(
        ptr(r_), ptr(w_), ptr(k_), ptr(v_), ptr(kk_), ptr(a_), ptr(state_c), ptr(new_state), ptr(g_), ptr(rk_),
        ptr(gw_), ptr(gb_), ptr(out), B, H, N, float(eps), dt_code(r_), _w_flag(w_, r_.dtype), stream_ptr(r_)),
        "fused_recurrent_output_prepare")
    return (out.reshape(B, H * N) if flat else out.reshape(B, H, N)), new_state


def fused_recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, state, g, k_k, k_a, r_k, group_norm_weight,
                                       group_norm_bias, *, eps: float, block_n: int = 64, num_warps: int = 8,
                                       force_fallback: bool = False, out=None, new_state=None, w_bias=None,
                                       a_bias=None, a_is_raw: bool = False, v_first=None, v_gate=None,
                                       v_gate_bias=None, v_gate_is_raw: bool = False, v_out=None,
                                       state_prefetch: bool = False, elapsed=None, advance_elapsed: bool = False,
                                       slot_ids=None):
    """Decode recurrence / output prep straight from raw w, k and sigmoid(a).

    The keyword arguments after ``force_fallback`` are extensions of this package (the reference
    signature ends there): they fold the LoRA biases, the sigmoid of ``a`` and of the v gate and
    the ``v_first`` interpolation into the same kernel, and allow in-place operation by passing
    ``new_state=state``.  ``state_prefetch=True`` lets the kernel load its state tile before it waits for the
    kernel that precedes it in the stream: only for call sequences in which that kernel never writes ``state``
    (a decode step, where a projection precedes the recurrence).  A float16 ``state`` selects the FP16-state lane
    (fp32 arithmetic, state rounded on the store); ``elapsed`` (int32 ``[B]``) adds the decay dither of the reference's
    native_wkv_fp16 extension and ``advance_elapsed`` increments it after the step.  ``slot_ids`` (int32 ``[B]``):
    ``state`` is a pool ``[capacity,H,N,N]`` (fp32) updated in place at rows ``slot_ids[b]``, and ``v_first`` / ``v_out``
    are pools ``[capacity, H*N]`` indexed the same way; the returned state is the pool."""
    no_fallback(force_fallback, "fused_recurrent_output_prepare_raw")
    if slot_ids is not None:
        return _output_prepare_raw_pool(r, w_raw, k_raw, v, a, state, g, k_k, k_a, r_k, group_norm_weight, group_norm_bias,
                                        float(eps), out, w_bias, a_bias, a_is_raw, v_first, v_gate, v_gate_bias,
                                        v_gate_is_raw, v_out, state_prefetch, slot_ids)
    B, H, N = _state_shape(state, allow_f16=True)
    if elapsed is not None:
        if state.dtype != torch.float16:
            raise ValueError("elapsed (decay dither) belongs to the float16-state lane")
        if not (elapsed.is_cuda and elapsed.dtype == torch.int32 and elapsed.is_contiguous() and int(elapsed.numel()) == B):
            raise ValueError("elapsed must be a contiguous CUDA int32 [B] tensor")
    elif advance_elapsed:
        raise ValueError("advance_elapsed needs elapsed")
    if int(block_n) < N:
        raise ValueError(f"block_n must be >= head_dim={N}; got {block_n}")
    if int(num_warps) not in {1, 2, 4, 8}:
        raise ValueError(f"num_warps must be one of 1, 2, 4, or 8; got {num_warps}")
    r_, flat = _as_bhn(r, B, H, N, "r")
    w_, k_, v_, a_, g_ = (_as_bhn(t, B, H, N, n)[0] for t, n in
                          ((w_raw, "w_raw"), (k_raw, "k_raw"), (v, "v"), (a, "a"), (g, "g")))
    hidden = H * N
    for value, name in ((k_k, "k_k"), (k_a, "k_a"), (r_k, "r_k"), (group_norm_weight, "group_norm_weight"),
                        (group_norm_bias, "group_norm_bias")):
        if int(value.numel()) != hidden:
            raise ValueError(f"{name} must contain {hidden} values")
    params = [t.contiguous() for t in (k_k, k_a, r_k, group_norm_weight, group_norm_bias)]
    opt = [None if t is None else t.contiguous() for t in (w_bias, a_bias, v_first, v_gate, v_gate_bias)]
    require_cuda(r_, w_, k_, v_, a_, g_, state, *params, *opt, what="fused_recurrent_output_prepare_raw")
    same_dtype(r_, w_, k_, v_, a_, g_, *params, *opt, what="fused_recurrent_output_prepare_raw")
    state_c = state.contiguous()
    if new_state is None:
        new_state = torch.empty_like(state_c)
    if out is None:
        out = torch.empty_like(r_)
    head = (ptr(r_), ptr(w_), ptr(k_), ptr(v_), ptr(a_), ptr(state_c), ptr(new_state), ptr(g_), ptr(params[0]),
            ptr(params[1]), ptr(params[2]), ptr(params[3]), ptr(params[4]), ptr(out), ptr(opt[0]), ptr(opt[1]),
            int(bool(a_is_raw)), ptr(opt[2]), ptr(opt[3]), ptr(opt[4]), int(bool(v_gate_is_raw)), ptr(v_out))
    tail = (int(bool(state_prefetch)), B, H, N, float(eps), dt_code(r_), stream_ptr(r_))
    if state_c.dtype == torch.float32:
        _lib.check(_lib.lib.rwkv7_wkv7_output_prepare_raw(*head, *tail), "fused_recurrent_output_prepare_raw")
    else:
        _lib.check(_lib.lib.rwkv7_wkv7_output_prepare_raw_f16state(*head, ptr(elapsed), int(bool(advance_elapsed)), *tail),
                   "fused_recurrent_output_prepare_raw", kernels=2 if advance_elapsed else 1)
    return (out.reshape(B, hidden) if flat else out.reshape(B, H, N)), new_state


def _output_prepare_raw_pool(r, w_raw, k_raw, v, a, pool, g, k_k, k_a, r_k, gn_w, gn_b, eps, out, w_bias, a_bias, a_is_raw,
                             v_first, v_gate, v_gate_bias, v_gate_is_raw, v_out, state_prefetch, slot_ids):
    _, H, N = _state_shape(pool, allow_f16=False)
    B = int(slot_ids.numel())
    if not (slot_ids.is_cuda and slot_ids.dtype == torch.int32 and slot_ids.is_contiguous()):
        raise ValueError("slot_ids must be a contiguous CUDA int32 tensor")
    if not pool.is_contiguous():
        raise ValueError("the state pool must be contiguous (it is updated in place)")
    r_, flat = _as_bhn(r, B, H, N, "r")
    w_, k_, v_, a_, g_ = (_as_bhn(t, B, H, N, n)[0] for t, n in
                          ((w_raw, "w_raw"), (k_raw, "k_raw"), (v, "v"), (a, "a"), (g, "g")))
    hidden = H * N
    for value, name in ((k_k, "k_k"), (k_a, "k_a"), (r_k, "r_k"), (gn_w, "group_norm_weight"), (gn_b, "group_norm_bias")):
        if int(value.numel()) != hidden:
            raise ValueError(f"{name} must contain {hidden} values")
    for value, name in ((v_first, "v_first"), (v_out, "v_out")):
        if value is not None and (value.dim() != 2 or int(value.shape[1]) != hidden or int(value.shape[0]) != int(pool.shape[0])
                                  or not value.is_contiguous()):
            raise ValueError(f"with slot_ids, {name} must be a contiguous pool [capacity, {hidden}]")
    params = [t.contiguous() for t in (k_k, k_a, r_k, gn_w, gn_b)]
    opt = [None if t is None else t.contiguous() for t in (w_bias, a_bias, v_gate, v_gate_bias)]
    require_cuda(r_, w_, k_, v_, a_, g_, pool, *params, *opt, v_first, v_out, what="fused_recurrent_output_prepare_raw")
    same_dtype(r_, w_, k_, v_, a_, g_, *params, *opt, v_first, v_out, what="fused_recurrent_output_prepare_raw")
    if out is None:
        out = torch.empty_like(r_)
    _lib.check(_lib.lib.rwkv7_wkv7_output_prepare_raw_pool(
        ptr(r_), ptr(w_), ptr(k_), ptr(v_), ptr(a_), ptr(pool), ptr(slot_ids), ptr(g_), ptr(params[0]), ptr(params[1]),
        ptr(params[2]), ptr(params[3]), ptr(params[4]), ptr(out), ptr(opt[0]), ptr(opt[1]), int(bool(a_is_raw)),
        ptr(v_first), ptr(opt[2]), ptr(opt[3]), int(bool(v_gate_is_raw)), ptr(v_out), int(bool(state_prefetch)), B, H, N,
        eps, dt_code(r_), stream_ptr(r_)), "fused_recurrent_output_prepare_raw")
    return (out.reshape(B, hidden) if flat else out.reshape(B, H, N)), pool


def _scan(name, r, w, k, v, kk, a, state, w_mode, prep=None, eps=0.0, chunk=0, ab_mode=False, w0=None, elapsed=None,
          new_state=None):
    B, H, N = _state_shape(state, allow_f16=not chunk)
    r_, flat = _as_bthn(r, B, H, N, "r")
    T = int(r_.shape[1])
    w_, k_, v_, kk_, a_ = (_as_bthn(t, B, H, N, n)[0] for t, n in ((w, "w"), (k, "k"), (v, "v"), (kk, "kk"), (a, "a")))
    for t, n in ((w_, "w"), (k_, "k"), (v_, "v"), (kk_, "kk"), (a_, "a")):
        if int(t.shape[1]) != T:
            raise ValueError(f"{n} must have {T} tokens")
    require_cuda(r_, w_, k_, v_, kk_, a_, state, what=name)
    same_dtype(r_, k_, v_, kk_, a_, what=name)
    if w_mode == 0:
        w_mode = _w_flag(w_, r_.dtype)
    elif w_.dtype != r_.dtype:
        raise ValueError("raw w must have the activation dtype")
    state_c = state.contiguous()
    if new_state is None:
        new_state = torch.empty_like(state_c)
    out = torch.empty_like(r_)
    if chunk:
        _lib.check(_lib.lib.rwkv7_wkv7_chunk_scan(ptr(r_), ptr(w_), ptr(k_), ptr(v_), ptr(kk_), ptr(a_), ptr(state_c),
                                                  ptr(new_state), ptr(out), B, T, H, N, int(chunk), dt_code(r_),
                                                  w_mode, stream_ptr(r_)), name)
    else:
        g_ = rk_ = gw_ = gb_ = None
        if prep is not None:
            g, r_k, gn_w, gn_b = prep
            g_ = _as_bthn(g, B, H, N, "g")[0]
            _check_prep_params(H, N, r_k, gn_w, gn_b)
            rk_, gw_, gb_ = r_k.contiguous(), gn_w.contiguous(), gn_b.contiguous()
            require_cuda(g_, rk_, gw_, gb_, what=name)
            same_dtype(r_, g_, rk_, gw_, gb_, what=name)
        if state_c.dtype == torch.float32 and not (ab_mode or w0 is not None or elapsed is not None):
            _lib.check(_lib.lib.rwkv7_wkv7_scan(ptr(r_), ptr(w_), ptr(k_), ptr(v_), ptr(kk_), ptr(a_), ptr(state_c),
                                                ptr(new_state), ptr(out), ptr(g_), ptr(rk_), ptr(gw_), ptr(gb_),
                                                float(eps), B, T, H, N, dt_code(r_), w_mode, stream_ptr(r_)), name)
        else:
            if state_c.dtype != torch.float16:
                raise ValueError(f"{name}: the neg_kk / kka / w0 / elapsed operand forms belong to the float16-state lane")
            _lib.check(_lib.lib.rwkv7_wkv7_scan_f16state(
                ptr(r_), ptr(w_), ptr(k_), ptr(v_), ptr(kk_), ptr(a_), ptr(state_c), ptr(new_state), ptr(out), ptr(g_),
                ptr(rk_), ptr(gw_), ptr(gb_), float(eps), B, T, H, N, dt_code(r_), w_mode, int(bool(ab_mode)), ptr(w0),
                ptr(elapsed), stream_ptr(r_)), name)
    return (out.reshape(B, T, H * N) if flat else out), new_state


def fused_recurrent_scan(r, w, k, v, kk, a, state, *, block_n: int = 64, block_m: int = 0, num_warps: int = 0,
                         force_fallback: bool = False):
    """T-token sequential scan; ``w`` is the decay.  Returns ``(out [B,T,...], final_state)``."""
    no_fallback(force_fallback, "fused_recurrent_scan")
    return _scan("fused_recurrent_scan", r, w, k, v, kk, a, state, 0)


def fused_recurrent_scan_clampw(r, w_raw, k, v, kk, a, state, *, block_n: int = 64, block_m: int = 0,
                                num_warps: int = 0, force_fallback: bool = False):
    """Scan that takes raw w and computes ``exp(-0.606531*sigmoid(w_raw))`` in-kernel."""
    no_fallback(force_fallback, "fused_recurrent_scan_clampw")
    return _scan("fused_recurrent_scan_clampw", r, w_raw, k, v, kk, a, state, 2)


def fused_recurrent_scan_output_prepare(r, w, k, v, kk, a, state, g, r_k, group_norm_weight, group_norm_bias, *,
                                        eps: float, block_n: int = 64, num_warps: int = 8,
                                        force_fallback: bool = False):
    """Scan + per-token GroupNorm / bonus / gate."""
    no_fallback(force_fallback, "fused_recurrent_scan_output_prepare")
    return _scan("fused_recurrent_scan_output_prepare", r, w, k, v, kk, a, state, 0,
                 prep=(g, r_k, group_norm_weight, group_norm_bias), eps=eps)


def fused_recurrent_scan_state_prep(r, w_raw, k_raw, v_raw, a, state, k_k, k_a, *, v_first=None, v_gate=None,
                                    block_n: int = 64, block_m=None, num_warps=None, force_fallback: bool = False):
    """State prep folded into the scan (rwkv7_hf/fused_recurrent_update.py:1541): raw w / k / v and sigmoided a / v-gate
    in, ``(out, final_state, k_adjusted, v_interpolated)`` out.  Two launches: the K / V / KK prep kernel, then the
    scan kernel, which computes the decay from raw w itself."""
    from . import prep as _prep
    no_fallback(force_fallback, "fused_recurrent_scan_state_prep")
    B, H, N = _state_shape(state)
    if int(block_n) < N:
        raise ValueError(f"block_n must be >= head_dim={N}; got {block_n}")
    if block_m is not None and not 0 < int(block_m) <= N:
        raise ValueError(f"block_m must be in [1, head_dim={N}]; got {block_m}")
    if num_warps is not None and int(num_warps) not in {1, 2, 4, 8}:
        raise ValueError(f"num_warps must be one of 1, 2, 4, or 8; got {num_warps}")
    hidden = H * N
    if int(k_k.numel()) != hidden or int(k_a.numel()) != hidden:
        raise ValueError(f"k_k and k_a must have {hidden} elements")
    r4, flat = _as_bthn(r, B, H, N, "r")
    T = int(r4.shape[1])
    as3 = lambda t, n: None if t is None else _as_bthn(t, B, H, N, n)[0].reshape(B, T, hidden)
    k, v, kk = _prep.fused_prefill_kv_kk_prep(as3(k_raw, "k_raw"), as3(v_raw, "v_raw"), as3(a, "a"), k_k, k_a,
                                              v_first=as3(v_first, "v_first"), v_gate=as3(v_gate, "v_gate"),
                                              num_heads=H, head_dim=N)
    out, final = _scan("fused_recurrent_scan_state_prep", r4, as3(w_raw, "w_raw"), k, v, kk, as3(a, "a"), state, 2)
    shape = (B, T, hidden) if flat else (B, T, H, N)
    return out.reshape(shape), final, k.reshape(shape), v.reshape(shape)


def self_chunk_rwkv7(r, w_decay, k, v, kk, a_gate, state_native, *, chunk_size: int = 16, w_is_log: bool = False,
                     safe_gate=None, h_tiles=None, w_is_raw: bool = False):
    """Chunked WY/DPLR scan on tensor cores (rwkv7_hf/self_chunk_rwkv7.py:33).  ``T`` must be a
    multiple of ``chunk_size`` and the head size 64, as in the reference (:56-62).  ``w_is_raw`` (an extension):
    ``w_decay`` holds the raw decay logits and the kernel forms ``exp(-0.606531 * sigmoid(w))`` itself, as the
    reference's clamp-w scans do (rwkv7_hf/fused_recurrent_update.py:1420), so no decay tensor is materialised."""
    if w_is_raw:
        if w_is_log:
            raise ValueError("w_is_raw and w_is_log exclude each other")
        T = int(r.shape[1])
        if chunk_size not in (16, 32, 64) or T % int(chunk_size):
            raise ValueError(f"self_chunk_rwkv7 requires chunk_size in (16, 32, 64) dividing T={T}; got {chunk_size}")
        return _scan("self_chunk_rwkv7", r, w_decay, k, v, kk, a_gate, state_native, 2,
                     chunk=int(chunk_size) if r.dtype == torch.float16 else 0)
    if w_is_log:
        w_decay = torch.exp(w_decay.float())
    T = int(r.shape[1])
    if chunk_size not in (16, 32, 64) or T % int(chunk_size):
        raise ValueError(f"self_chunk_rwkv7 requires chunk_size in (16, 32, 64) dividing T={T}; got {chunk_size}")
    if r.dtype != torch.float16:  # the tensor-core kernel is fp16 only; the sequential kernel computes the same scan
        return _scan("self_chunk_rwkv7", r, w_decay, k, v, kk, a_gate, state_native, 0)
    return _scan("self_chunk_rwkv7", r, w_decay, k, v, kk, a_gate, state_native, 0, chunk=int(chunk_size))


def dplr_chunk_scan(r, w, k, v, kk, a, state, *, chunk_size: int = 64, force_fallback: bool = False, algorithm=None):
    """rwkv7_hf/dplr_prefill.py:505: any positive chunk size; the result does not depend on it.
    Chunk sizes the tensor-core kernel takes (16/32/64 dividing T) use it, others run the
    sequential kernel, which computes the same recurrence."""
    no_fallback(force_fallback, "dplr_chunk_scan")
    if int(chunk_size) <= 0:
        raise ValueError("chunk_size must be positive")
    T = int(r.shape[1])
    if algorithm in ("wy", "lowrank", "cuda_wy") and chunk_size in (16, 32, 64) and T % chunk_size == 0 and T > 0 \
            and r.dtype == torch.float16:  # the tensor-core kernel is fp16 only
        return _scan("dplr_chunk_scan", r, w, k, v, kk, a, state, 0, chunk=int(chunk_size))
    return _scan("dplr_chunk_scan", r, w, k, v, kk, a, state, 0)


# ------------------------------------------------------------------ FP16-state lane of the native_wkv_fp16 extension
def native_fp16_recurrent_should_use(*, state_dtype, input_dtype, head_dim: int) -> bool:
    """rwkv7_hf/native_wkv_fp16.py:597-608."""
    return bool(state_dtype == torch.float16 and input_dtype == torch.float16 and int(head_dim) == 64)


def native_fp16_recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, state, g, k_k, k_a, r_k, norm_weight, norm_bias,
                                             elapsed, *, advance_elapsed: bool, eps: float):
    """Decode step on an fp16 ``state [B,H,64,64]`` updated IN PLACE, with the decay dither phased by ``elapsed``
    (int32 ``[B]``; incremented when ``advance_elapsed``).  Same signature, argument checks and return value (the
    prepared output) as rwkv7_hf/native_wkv_fp16.py:678-770."""
    if state.dim() != 4:
        raise ValueError("state must be [B,H,64,64]")
    if not native_fp16_recurrent_should_use(state_dtype=state.dtype, input_dtype=r.dtype, head_dim=int(state.shape[-1])):
        raise ValueError("native FP16 recurrence received an unsupported dtype or shape")
    tensors = (r, w_raw, k_raw, v, a, state, g, k_k, k_a, r_k, norm_weight, norm_bias)
    if not all(t.is_cuda and t.dtype == torch.float16 and t.is_contiguous() for t in tensors):
        raise ValueError("native FP16 recurrence requires contiguous CUDA fp16 tensors")
    if not (elapsed.is_cuda and elapsed.dtype == torch.int32 and elapsed.is_contiguous()):
        raise ValueError("elapsed must be a contiguous CUDA int32 tensor")
    out, _ = fused_recurrent_output_prepare_raw(r, w_raw, k_raw, v, a, state, g, k_k, k_a, r_k, norm_weight, norm_bias,
                                                eps=float(eps), new_state=state, elapsed=elapsed,
                                                advance_elapsed=bool(advance_elapsed))
    return out


def native_fp16_sequence(r, w, k, v, neg_kk, kka, state, elapsed, *, w0=None):
    """FP16-state scan over ``[B,T,H,64]`` (rwkv7_hf/native_wkv_fp16.py:773-821): ``w`` is the raw decay input (``w0`` is
    added to it when given), ``neg_kk = -kk``, ``kka = kk*a``; ``state`` is updated in place; token ``t`` uses the dither
    phase ``elapsed + t``.  Returns the recurrent output in the layout of ``r``."""
    if state.dim() != 4 or r.dim() != 4:
        raise ValueError("state and sequence tensors must be rank four")
    if not native_fp16_recurrent_should_use(state_dtype=state.dtype, input_dtype=r.dtype, head_dim=int(state.shape[-1])):
        raise ValueError("native FP16 sequence received an unsupported dtype or shape")
    if not all(t.is_cuda and t.dtype == torch.float16 and t.is_contiguous() for t in (r, w, k, v, neg_kk, kka, state)):
        raise ValueError("native FP16 sequence requires contiguous CUDA fp16 tensors")
    if not (elapsed.is_cuda and elapsed.dtype == torch.int32 and elapsed.is_contiguous()
            and int(elapsed.numel()) == int(r.shape[0])):
        raise ValueError("elapsed must be a contiguous CUDA int32 [B] tensor")
    if w0 is not None and not (w0.is_cuda and w0.dtype == torch.float16 and w0.is_contiguous()):
        raise ValueError("w0 must be contiguous CUDA fp16")
    out, _ = _scan("native_fp16_sequence", r, w, k, v, neg_kk, kka, state, 2, ab_mode=True, w0=w0, elapsed=elapsed,
                   new_state=state)
    return out
