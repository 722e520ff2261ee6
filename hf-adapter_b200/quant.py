"""Quantised projections: formats, free functions and ``nn.Linear`` replacements.

Formats and names follow the reference so packed buffers are interchangeable:

* int8 per-output-channel ("MM8"): ``quantize_w8_row`` / ``w8_linear``
  (rwkv7_hf/sm70_quant.py:485-489,522) and ``MM8Linear`` with buffers ``q_row [out,in] i8``,
  ``row_scale [out]`` (rwkv7_hf/native_quant_mm8.py:577-580).
* int4 group-128/256 ("MM4"): ``quantize_w4_groupwise`` / ``w4_groupwise_linear``
  (rwkv7_hf/sm70_quant.py:502-519,579) and ``MM4Linear(group_size=128)`` with buffers
  ``packed_group [out,in/2] u8``, ``group_scales [out,in/group]`` (rwkv7_hf/native_quant_mm4.py:601-607);
  an optional ``group_zeros [out,in/group] u8`` buffer generalises the implicit zero-point 8.
* A8W8: ``quantize_weight_per_channel_int8`` / ``a8w8_linear`` / ``A8W8Linear`` with buffers
  ``q_weight_t [in,out] i8`` and ``weight_scale [out] fp32`` (rwkv7_hf/native_quant_a8w8.py:312-571).

The quantisers are load-time tensor code (plain torch, any device).  Every forward runs on the
CUDA library; there is no CPU forward.
"""
from __future__ import annotations

import torch

from . import _lib
from ._util import dt_code, ptr, require_cuda, stream_ptr

GEMV_MAX_ROWS = 64  # rows up to which the weight-streaming kernels are used; above: dequantise + GEMM
TILED_MAX_ROWS = 512  # rows up to which MM4Linear uses the tensor-core decode kernel (one weight pass per 64 rows)


# ------------------------------------------------------------------ quantisers (load time)
def quantize_w8_row(weight):
    w = weight.detach().float()
    s = (w.abs().amax(1) / 127).clamp_min(1e-6)
    q = (w / s[:, None]).round().clamp(-127, 127).to(torch.int8)
    return q.contiguous(), s.to(weight.dtype)


def quantize_w4_groupwise(weight, group_size=128):
    group_size = int(group_size)
    if group_size not in {128, 256}:
        raise ValueError("groupwise W4 requires group_size=128 or 256")
    if weight.dim() != 2 or weight.shape[1] % group_size:
        raise ValueError("groupwise W4 requires rank-2 weight with K divisible by group_size")
    w = weight.detach().float()
    out_features, in_features = w.shape
    grouped = w.reshape(out_features, in_features // group_size, group_size)
    scales = (grouped.abs().amax(dim=2) / 7).clamp_min(1e-6)
    q = (grouped / scales[:, :, None]).round().clamp(-7, 7).to(torch.int16) + 8
    q = q.reshape(out_features, in_features)
    packed = ((q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)).contiguous()
    return packed, scales.to(weight.dtype).contiguous(), in_features


def quantize_weight_per_channel_int8(weight):
    """Returns ``(q_weight_t [in,out] int8, scales [out] fp32)``.  ``q_weight_t`` is the transposed VIEW of a
    contiguous ``[out,in]`` tensor: same values and shape as the reference's buffer, K-major in memory,
    which is the operand layout the tensor-core GEMM reads."""
    fp32 = weight.detach().float()
    scales = (fp32.abs().amax(dim=1) / 127.0).clamp_min(1.0e-5)
    quantized = (fp32 / scales[:, None]).round().clamp(-127, 127).to(torch.int8).contiguous()
    return quantized.t(), scales.contiguous()


# ------------------------------------------------------------------ free functions
def _rows(x, K):
    if int(x.shape[-1]) != K:
        raise ValueError(f"input must end in {K} features; got {tuple(x.shape)}")
    return x.reshape(-1, K).contiguous()


def _epi(relu2, residual, M, Nout, x2):
    if relu2 and residual is not None:
        raise ValueError("choose one epilogue")
    if residual is not None:
        res = residual.reshape(M, Nout).contiguous()
        require_cuda(res, what="quant linear")
        if res.dtype != x2.dtype:
            raise ValueError("residual dtype must match the activations")
        return _lib.EPI_ADD, res
    return (_lib.EPI_RELU2 if relu2 else _lib.EPI_NONE), None


def w4_dequant(q, scales, in_features, group_size=128, zeros=None, out=None):
    """Dense ``[out,in]`` weight in the dtype of ``scales``."""
    Nout = int(q.shape[0])
    require_cuda(q, scales, zeros, what="w4_dequant")
    if out is None:
        out = torch.empty((Nout, int(in_features)), device=q.device, dtype=scales.dtype)
    _lib.check(_lib.lib.rwkv7_w4g_dequant(ptr(q), ptr(scales), ptr(zeros), ptr(out), int(in_features), Nout,
                                          int(group_size), dt_code(scales), stream_ptr(q)), "w4_dequant")
    return out


def w4_repack_tiled(q, scales, in_features, group_size=128, zeros=None):
    """Build the tiled copy of a group-wise int4 weight that the tensor-core decode kernel streams (one 8704-byte
    block per [128 channels x 128 k] tile: nibbles, scales, zero-points).  Returns one uint8 tensor.  Done once at
    load time; the reference-layout tensors stay the interchange format."""
    Nout, K = int(q.shape[0]), int(in_features)
    require_cuda(q, scales, zeros, what="w4_repack_tiled")
    if scales.dtype != torch.float16:
        raise ValueError("the tiled format holds fp16 scales")
    nbytes = int(_lib.lib.rwkv7_w4g_tiled_bytes(K, Nout))
    if nbytes == 0:
        raise ValueError(f"in_features={K} is not a multiple of 128")
    tiled = torch.empty((nbytes,), device=q.device, dtype=torch.uint8)
    _lib.check(_lib.lib.rwkv7_w4g_repack(ptr(q.contiguous()), ptr(scales.contiguous()), ptr(zeros), ptr(tiled),
                                         K, Nout, int(group_size), _lib.F16, stream_ptr(q)), "w4_repack_tiled")
    return tiled


def w4_tiled_linear(x, tiled, out_features, in_features, *, out=None, relu2: bool = False, residual=None):
    """y = x @ W^T on the tensor-core kernel from the tiled weight copy (fp16; one weight pass per 64 rows)."""
    K, Nout = int(in_features), int(out_features)
    x2 = _rows(x, K)
    M = int(x2.shape[0])
    require_cuda(x2, tiled, what="w4_tiled_linear")
    epi, res = _epi(relu2, residual, M, Nout, x2)
    y = torch.empty((M, Nout), device=x2.device, dtype=x2.dtype) if out is None else out.reshape(M, Nout)
    _lib.check(_lib.lib.rwkv7_w4g_gemv_tiled(ptr(x2), ptr(tiled), ptr(res), ptr(y), M, K, Nout, epi, dt_code(x2),
                                             stream_ptr(x2)), "w4_tiled_linear")
    return y.reshape(*x.shape[:-1], Nout)


def w4_tiled_linear_group(xs, tileds, out_features, in_features, *, relu2: bool = False):
    """Up to four projections of the same shape in ONE launch of the tensor-core kernel: ``ys[g] = xs[g] @ W_g^T``
    (the r / k / v projections of a layer).  Returns the list of outputs."""
    import ctypes
    K, Nout, G = int(in_features), int(out_features), len(xs)
    if not 1 <= G <= 4 or len(tileds) != G:
        raise ValueError("w4_tiled_linear_group takes 1..4 activations and as many tiled weights")
    x2 = [_rows(x, K).contiguous() for x in xs]
    M = int(x2[0].shape[0])
    if any(int(t.shape[0]) != M or t.dtype != x2[0].dtype for t in x2):
        raise ValueError("grouped projections need the same row count and dtype")
    require_cuda(*x2, *tileds, what="w4_tiled_linear_group")
    ys = [torch.empty((M, Nout), device=x2[0].device, dtype=x2[0].dtype) for _ in range(G)]
    arr = lambda ts: (ctypes.c_void_p * G)(*[t.data_ptr() for t in ts])
    _lib.check(_lib.lib.rwkv7_w4g_gemv_tiled_group(arr(x2), arr(tileds), arr(ys), G, M, K, Nout, _lib.EPI_RELU2 if relu2 else
                                                   _lib.EPI_NONE, dt_code(x2[0]), stream_ptr(x2[0])), "w4_tiled_linear_group")
    return [y.reshape(*x.shape[:-1], Nout) for y, x in zip(ys, xs)]


def w8_repack_tiled(q):
    """Tiled copy of an int8 per-output-channel weight ``q [out,in]`` for the tensor-core kernel (16 KiB blocks of
    [128 channels x 128 k], bytes stored as q + 128).  Done once at load time."""
    Nout, K = (int(v) for v in q.shape)
    require_cuda(q, what="w8_repack_tiled")
    nbytes = int(_lib.lib.rwkv7_w8_tiled_bytes(K, Nout))
    if nbytes == 0:
        raise ValueError(f"in_features={K} is not a multiple of 128")
    tiled = torch.empty((nbytes,), device=q.device, dtype=torch.uint8)
    _lib.check(_lib.lib.rwkv7_w8_repack(ptr(q.contiguous()), ptr(tiled), K, Nout, stream_ptr(q)), "w8_repack_tiled")
    return tiled


def w8_tiled_linear_group(xs, tileds, scales, out_features, in_features, *, relu2: bool = False, residual=None, out=None):
    """``ys[g] = epilogue(xs[g] @ (q_g * s_g)^T)`` for up to four int8 projections of one shape in one launch of the
    tensor-core kernel (fp16).  ``residual`` / ``out`` apply to a single projection.  Returns the list of outputs."""
    import ctypes
    K, Nout, G = int(in_features), int(out_features), len(xs)
    if not 1 <= G <= 4 or len(tileds) != G or len(scales) != G:
        raise ValueError("w8_tiled_linear_group takes 1..4 activations and as many tiled weights and scales")
    x2 = [_rows(x, K) for x in xs]
    M = int(x2[0].shape[0])
    if any(int(t.shape[0]) != M or t.dtype != x2[0].dtype for t in x2):
        raise ValueError("grouped projections need the same row count and dtype")
    sc = [s.contiguous() for s in scales]
    require_cuda(*x2, *tileds, *sc, what="w8_tiled_linear_group")
    if any(s.dtype != x2[0].dtype or int(s.numel()) != Nout for s in sc):
        raise ValueError("scales must be [out_features] in the activation dtype")
    epi, res = _epi(relu2, residual, M, Nout, x2[0])
    if (res is not None or out is not None) and G != 1:
        raise ValueError("residual / out apply to a single projection")
    ys = [torch.empty((M, Nout), device=x2[0].device, dtype=x2[0].dtype) if out is None else out.reshape(M, Nout) for _ in range(G)]
    arr = lambda ts: (ctypes.c_void_p * G)(*[t.data_ptr() for t in ts])
    _lib.check(_lib.lib.rwkv7_w8_gemv_tiled_group(arr(x2), arr(tileds), arr(sc), ptr(res), arr(ys), G, M, K, Nout, epi,
                                                   dt_code(x2[0]), stream_ptr(x2[0])), "w8_tiled_linear_group")
    return [y.reshape(*x.shape[:-1], Nout) for y, x in zip(ys, xs)]


def w8_dequant(q, s, out=None):
    Nout, K = (int(v) for v in q.shape)
    require_cuda(q, s, what="w8_dequant")
    if out is None:
        out = torch.empty((Nout, K), device=q.device, dtype=s.dtype)
    _lib.check(_lib.lib.rwkv7_w8_dequant(ptr(q), ptr(s), ptr(out), K, Nout, dt_code(s), stream_ptr(q)), "w8_dequant")
    return out


def _dense_after_dequant(x2, weight, relu2, res, out):
    """Many rows over a quantised weight: the weight was materialised in the activation type as ``[out,in]``; one launch
    of this library's tensor-core GEMM applies it with the relu^2 / residual epilogue fused (fp16 / bf16; fp32
    activations take a library GEMM and pointwise kernels)."""
    from . import gemm as _gemm
    M, Nout = int(x2.shape[0]), int(weight.shape[0])
    if _gemm.takes(x2, weight):
        return _gemm.dense_linear(x2, weight, relu2=relu2, residual=res, out=None if out is None else out.reshape(M, Nout))
    y = torch.matmul(x2, weight.t())
    if relu2:
        y = torch.relu(y) ** 2
    elif res is not None:
        y = y + res
    if out is not None:
        out.reshape(M, Nout).copy_(y)
        y = out.reshape(M, Nout)
    return y


def w4_groupwise_linear(x, q, scales, out_features, in_features, *, group_size=128, out=None, zeros=None,
                        relu2: bool = False, residual=None):
    """y = x @ ((nibble - zero) * scale)^T.  Up to GEMV_MAX_ROWS rows run the weight-streaming kernel with the
    optional relu^2 / residual-add epilogue fused; more rows dequantise the weight and run this library's dense GEMM
    with the same epilogues (the reference dequantises and calls F.linear on every call off sm_70,
    rwkv7_hf/sm70_quant.py:598-610)."""
    group_size = int(group_size)
    if group_size not in {128, 256} or int(in_features) % group_size:
        raise ValueError("groupwise W4 requires group_size=128/256 and divisible K")
    K, Nout = int(in_features), int(out_features)
    x2 = _rows(x, K)
    M = int(x2.shape[0])
    require_cuda(x2, q, scales, zeros, what="w4_groupwise_linear")
    if scales.dtype != x2.dtype:
        raise ValueError(f"scales dtype {scales.dtype} must match the activation dtype {x2.dtype}")
    epi, res = _epi(relu2, residual, M, Nout, x2)
    if M <= GEMV_MAX_ROWS:
        y = torch.empty((M, Nout), device=x2.device, dtype=x2.dtype) if out is None else out.reshape(M, Nout)
        _lib.check(_lib.lib.rwkv7_w4g_gemv(ptr(x2), ptr(q), ptr(scales), ptr(zeros), ptr(res), ptr(y), M, K, Nout,
                                           group_size, epi, dt_code(x2), stream_ptr(x2)), "w4_groupwise_linear")
    else:
        y = _dense_after_dequant(x2, w4_dequant(q, scales, K, group_size, zeros), relu2, res, out)
    return y.reshape(*x.shape[:-1], Nout)


def w8_linear(x, q, s, out=None, *, relu2: bool = False, residual=None):
    """y = x @ (q * s[:,None])^T for int8 per-output-channel weights ``q [out,in]``."""
    Nout, K = (int(v) for v in q.shape)
    x2 = _rows(x, K)
    M = int(x2.shape[0])
    require_cuda(x2, q, s, what="w8_linear")
    if s.dtype != x2.dtype:
        raise ValueError(f"scale dtype {s.dtype} must match the activation dtype {x2.dtype}")
    epi, res = _epi(relu2, residual, M, Nout, x2)
    if M <= GEMV_MAX_ROWS:
        y = torch.empty((M, Nout), device=x2.device, dtype=x2.dtype) if out is None else out.reshape(M, Nout)
        _lib.check(_lib.lib.rwkv7_w8_gemv(ptr(x2), ptr(q), ptr(s), ptr(res), ptr(y), M, K, Nout, epi, dt_code(x2),
                                          stream_ptr(x2)), "w8_linear")
    else:
        y = _dense_after_dequant(x2, w8_dequant(q, s), relu2, res, out)
    return y.reshape(*x.shape[:-1], Nout)


def dynamic_a8_quant(x):
    """Per-row int8 quantisation of ``x [rows,K]``: returns ``(q int8, scale fp32 [rows])``."""
    K = int(x.shape[-1])
    x2 = _rows(x, K)
    require_cuda(x2, what="dynamic_a8_quant")
    q = torch.empty(x2.shape, device=x2.device, dtype=torch.int8)
    s = torch.empty((x2.shape[0],), device=x2.device, dtype=torch.float32)
    _lib.check(_lib.lib.rwkv7_a8_quant(ptr(x2), ptr(q), ptr(s), int(x2.shape[0]), K, dt_code(x2), stream_ptr(x2)),
               "dynamic_a8_quant")
    return q, s


def int8_mm(qa, qw_row):
    """Bit-exact ``qa [M,K] i8 @ qw_row[N,K]^T -> [M,N] i32`` (the role of torch._int_mm in the reference)."""
    M, K = (int(v) for v in qa.shape)
    N = int(qw_row.shape[0])
    if int(qw_row.shape[1]) != K:
        raise ValueError("inner dimensions differ")
    require_cuda(qa, qw_row, what="int8_mm")
    qa, qw_row = qa.contiguous(), qw_row.contiguous()
    acc = torch.empty((M, N), device=qa.device, dtype=torch.int32)
    _lib.check(_lib.lib.rwkv7_i8_gemm(ptr(qa), ptr(qw_row), ptr(acc), M, K, N, stream_ptr(qa)), "int8_mm")
    return acc


def _k_major(q_weight_t):
    """[in,out] reference-shaped weight -> contiguous [out,in] (free when it is the transposed view this
    package creates)."""
    qw = q_weight_t.t()
    return qw if qw.is_contiguous() else qw.contiguous()


def a8w8_workspace(M, K, Nout, device):
    n = int(_lib.lib.rwkv7_a8w8_workspace_bytes(int(M), int(K), int(Nout)))
    return torch.empty((n,), device=device, dtype=torch.uint8)


def a8w8_linear(x, q_weight_t, weight_scale, bias=None, *, out=None, residual=None, workspace=None, relu2: bool = False):
    """Dynamic-A8 / W8 linear (rwkv7_hf/native_quant_a8w8.py:323): quantise rows, int8 GEMM with exact int32
    accumulators, dequantise (+bias, +residual).  ``relu2`` (an extension): relu(.)**2 of the rounded output instead of
    a residual, in the same epilogue."""
    K = int(q_weight_t.shape[0])
    Nout = int(q_weight_t.shape[1])
    x2 = _rows(x, K)
    M = int(x2.shape[0])
    if K % 16 or Nout % 8:
        raise ValueError("a8w8_linear requires in_features % 16 == 0 and out_features % 8 == 0")
    qw = _k_major(q_weight_t)
    require_cuda(x2, qw, weight_scale, bias, residual, what="a8w8_linear")
    if weight_scale.dtype != torch.float32:
        raise ValueError("weight_scale must be float32")
    res = None if residual is None else residual.reshape(M, Nout).contiguous()
    if workspace is None:
        workspace = a8w8_workspace(M, K, Nout, x2.device)
    y = torch.empty((M, Nout), device=x2.device, dtype=x2.dtype) if out is None else out.reshape(M, Nout)
    if relu2:
        if res is not None:
            raise ValueError("the relu^2 epilogue takes no residual")
        _lib.check(_lib.lib.rwkv7_a8w8_linear_relu2(ptr(x2), ptr(qw), ptr(weight_scale), ptr(bias), ptr(y), ptr(workspace),
                                                    int(workspace.numel()), M, K, Nout, dt_code(x2), stream_ptr(x2)),
                   "a8w8_linear", kernels=2 if M >= 64 else 3)
        return y.reshape(*x.shape[:-1], Nout)
    _lib.check(_lib.lib.rwkv7_a8w8_linear(ptr(x2), ptr(qw), ptr(weight_scale), ptr(bias), ptr(res), ptr(y),
                                          ptr(workspace), int(workspace.numel()), M, K, Nout, dt_code(x2),
                                          stream_ptr(x2)), "a8w8_linear", kernels=2 if M >= 64 else 3)
    return y.reshape(*x.shape[:-1], Nout)


def a8w8_ffn(x, up, down, residual):
    """Paired A8W8 ``up -> relu^2 -> down + residual`` with the hidden activation kept in int8
    (rwkv7_hf/native_quant_a8w8.py:436): quantise rows, int8 GEMM, one kernel that dequantises, applies the fp16
    relu^2 boundary and requantises per row, int8 GEMM, dequantise + residual.  Returns ``None`` when the pairing
    does not meet the reference's contract (callers then run the two linears)."""
    if not isinstance(up, A8W8Linear) or not isinstance(down, A8W8Linear):
        return None
    if (not x.is_cuda or x.dtype != torch.float16 or up.out_features != down.in_features
            or up.in_features != down.out_features or up.in_features > 4096 or up.in_features % 16
            or up.out_features % 16):
        return None
    K, F_, D = up.in_features, up.out_features, down.out_features
    x2 = _rows(x, K)
    M = int(x2.shape[0])
    res = residual.reshape(-1, D)
    if M < 1 or int(res.shape[0]) != M or not res.is_contiguous():
        return None
    dev = x2.device
    qa = torch.empty((M, K), device=dev, dtype=torch.int8)
    sa = torch.empty((M,), device=dev, dtype=torch.float32)
    acc1 = torch.empty((M, F_), device=dev, dtype=torch.int32)
    qh = torch.empty((M, F_), device=dev, dtype=torch.int8)
    sh = torch.empty((M,), device=dev, dtype=torch.float32)
    acc2 = torch.empty((M, D), device=dev, dtype=torch.int32)
    y = torch.empty((M, D), device=dev, dtype=x2.dtype)
    st, dt = stream_ptr(x2), dt_code(x2)
    L = _lib.lib
    _lib.check(L.rwkv7_a8_quant(ptr(x2), ptr(qa), ptr(sa), M, K, dt, st), "a8w8_ffn: quantise")
    _lib.check(L.rwkv7_i8_gemm(ptr(qa), ptr(_k_major(up.q_weight_t)), ptr(acc1), M, K, F_, st), "a8w8_ffn: up GEMM")
    _lib.check(L.rwkv7_a8w8_relu2_requant(ptr(acc1), ptr(sa), ptr(up.weight_scale), ptr(up.bias), ptr(qh), ptr(sh), M, F_,
                                          dt, st), "a8w8_ffn: relu2 + requantise")
    _lib.check(L.rwkv7_i8_gemm(ptr(qh), ptr(_k_major(down.q_weight_t)), ptr(acc2), M, F_, D, st), "a8w8_ffn: down GEMM")
    _lib.check(L.rwkv7_a8w8_dequant(ptr(acc2), ptr(sh), ptr(down.weight_scale), ptr(down.bias), ptr(res), ptr(y), M, D,
                                    dt, st), "a8w8_ffn: dequantise")
    return y.reshape(*x.shape[:-1], D)


# ------------------------------------------------------------------ affine 8-bit / 4-bit formats
AFFINE_GEMV_MAX_ROWS = 32  # up to four 8-row passes over the weight bytes; beyond that: dequantise + one GEMM


def _affine_quant(weight, levels):
    """Shared body of quantize_mm8 / quantize_mm4 (rwkv7_hf/native_quant_mm8.py:62-97, native_quant_mm4.py:77-108):
    ``weight`` [N(in), M(out)]; two-sided min subtraction and max scaling, ``floor(w * levels)``."""
    w = weight.float()
    n, m = w.shape
    eps = 1e-8
    if n > m:
        my = w.amin(dim=1, keepdim=True); w = w - my
        mx = w.amin(dim=0); w = w - mx
    else:
        mx = w.amin(dim=0); w = w - mx
        my = w.amin(dim=1, keepdim=True); w = w - my
    rx = w.amax(dim=0).clamp(min=eps); w = w / rx
    ry = w.amax(dim=1, keepdim=True).clamp(min=eps); w = w / ry
    q = torch.clamp(torch.floor(w * float(levels)), 0, levels - 1).to(torch.uint8)
    return q, mx, rx, my, ry


def quantize_mm8(weight):
    """``weight`` [N, M] -> ``(w_u8 [N,M], mx [M], rx [M], my [N,1], ry [N,1])`` in ``weight.dtype`` (fp16i8)."""
    q, mx, rx, my, ry = _affine_quant(weight, 256)
    od = weight.dtype
    return q, mx.to(od), (rx / 16.0).to(od), my.to(od), (ry / 16.0).to(od)


def quantize_mm4(weight):
    """``weight`` [N, M] -> ``(packed [N, Mp/2] u8, mx [Mp], rx_s [Mp], my [N,1], ry_s [N,1], M, Mp)``; low nibble =
    even output column, the output width padded to even."""
    m_orig = int(weight.shape[1])
    w = weight.float()
    if m_orig % 2:
        w = torch.nn.functional.pad(w, (0, 1))
    q, mx, rx, my, ry = _affine_quant(w, 16)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8).contiguous()
    od = weight.dtype
    return packed, mx.to(od), (rx / 4.0).to(od), my.to(od), (ry / 4.0).to(od), m_orig, int(w.shape[1])


def _affine_dequant(q, mx, rx, my, ry, Nout, bits, dtype):
    K = int(q.shape[0])
    require_cuda(q, mx, rx, my, ry, what="affine dequant")
    cast = lambda t: t.reshape(-1).to(dtype).contiguous()
    mx_, rx_, my_, ry_ = cast(mx), cast(rx), cast(my), cast(ry)
    W = torch.empty((K, Nout), device=q.device, dtype=dtype)
    _lib.check(_lib.lib.rwkv7_affine_dequant(ptr(q.contiguous()), ptr(mx_), ptr(rx_), ptr(my_), ptr(ry_), ptr(W), K, Nout,
                                             bits, dt_code(W), stream_ptr(q)), "affine dequant")
    return W


def dequantize_mm8(w_u8, mx, rx, my, ry, out_dtype=None):
    """The dequantised weight [N, M] with the reference's operation order and rounding (native_quant_mm8.py:100)."""
    return _affine_dequant(w_u8, mx, rx, my, ry, int(w_u8.shape[1]), 8, out_dtype if out_dtype is not None else mx.dtype)


def dequantize_mm4(packed, mx, rx_s, my, ry_s, m_orig, out_dtype=None):
    return _affine_dequant(packed, mx, rx_s, my, ry_s, int(m_orig), 4, out_dtype if out_dtype is not None else mx.dtype)


def _affine_matmul(x, q, mx, rx, my, ry, Nout, bits, what):
    K = int(q.shape[0])
    x2 = _rows(x, K)
    M = int(x2.shape[0])
    require_cuda(x2, q, mx, rx, my, ry, what=what)
    if M <= AFFINE_GEMV_MAX_ROWS and Nout % 8 == 0 and (bits == 8 or int(q.shape[1]) * 2 == Nout):
        dt = x2.dtype
        cast = lambda t: t.reshape(-1).to(dt).contiguous()
        mx_, rx_, my_, ry_ = cast(mx), cast(rx), cast(my), cast(ry)
        qc = q.contiguous()
        y = torch.empty((M, Nout), device=x2.device, dtype=dt)
        for m0 in range(0, M, 8):
            rows = min(8, M - m0)
            nbytes = int(_lib.lib.rwkv7_affine_gemv_workspace_bytes(rows, K, Nout))
            ws = torch.empty((nbytes // 4,), device=x2.device, dtype=torch.float32)
            _lib.check(_lib.lib.rwkv7_affine_gemv(ptr(x2[m0:m0 + rows]), ptr(qc), ptr(mx_), ptr(rx_), ptr(my_), ptr(ry_),
                                                  ptr(y[m0:m0 + rows]), ptr(ws), nbytes, rows, K, Nout, bits, dt_code(x2),
                                                  stream_ptr(x2)), what, kernels=2)
        return y.reshape(*x.shape[:-1], Nout)
    W = _affine_dequant(q, mx, rx, my, ry, Nout, bits, x2.dtype)  # many rows: materialise, then one library GEMM
    return (x2 @ W).reshape(*x.shape[:-1], Nout)


def mm8_matmul(x, w_u8, mx, rx, my, ry):
    """``y = x @ dequant(W)`` for ``x [..., N]`` (rwkv7_hf/native_quant_mm8.py:110, fused route :468): up to
    AFFINE_GEMV_MAX_ROWS rows stream the u8 weights through the GEMV kernel, more rows dequantise once and call a GEMM."""
    return _affine_matmul(x, w_u8, mx, rx, my, ry, int(w_u8.shape[1]), 8, "mm8_matmul")


def mm4_matmul(x, packed, mx, rx_s, my, ry_s, m_orig):
    """4-bit affine counterpart (rwkv7_hf/native_quant_mm4.py:128, fused route :545)."""
    return _affine_matmul(x, packed, mx, rx_s, my, ry_s, int(m_orig), 4, "mm4_matmul")


def mm8_matmul_triton(x, w_u8, mx, rx, my, ry, *, max_gemv_rows=None):
    """The reference's name for its fused route; here the CUDA kernels above."""
    return mm8_matmul(x, w_u8, mx, rx, my, ry)


def mm4_matmul_triton(x, packed, mx, rx_s, my, ry_s, m_orig, *, max_gemv_rows=None):
    return mm4_matmul(x, packed, mx, rx_s, my, ry_s, m_orig)


mm8_gemv_triton = mm8_matmul
mm4_gemv_triton = mm4_matmul


# ------------------------------------------------------------------ modules
class MM8Linear(torch.nn.Module):
    """``nn.Linear`` replacement with 8-bit weights.  Default: the reference's fp16i8 affine format (buffers ``w_u8``
    [in,out], ``mx``, ``rx`` [out], ``my``, ``ry`` [in,1]: what rwkv7_hf/native_quant_mm8.py:564-592 stores on devices
    other than sm7x).  ``rowwise=True``: per-output-channel symmetric int8 (buffers ``q_row``, ``row_scale``: its sm7x
    format), whose kernel fuses the relu^2 / residual epilogues."""

    def __init__(self, linear, *, fused=True, rowwise=False):
        super().__init__()
        self.in_features, self.out_features = int(linear.weight.shape[1]), int(linear.weight.shape[0])
        self.sm7x_rowwise = bool(rowwise)
        if self.sm7x_rowwise:
            q_row, row_scale = quantize_w8_row(linear.weight.data)
            self.register_buffer("q_row", q_row)
            self.register_buffer("row_scale", row_scale)
        else:
            wu8, mx, rx, my, ry = quantize_mm8(linear.weight.data.t().contiguous())
            self.register_buffer("w_u8", wu8)
            self.register_buffer("mx", mx)
            self.register_buffer("rx", rx)
            self.register_buffer("my", my)
            self.register_buffer("ry", ry)
        if linear.bias is not None:
            self.register_buffer("bias", linear.bias.data.clone())
        else:
            self.bias = None
        self.fused = bool(fused)
        self._tiled = None  # tiled copy of q_row for the tensor-core kernel (derived, not part of the state dict)

    def _load_from_state_dict(self, *args, **kwargs):
        self._tiled = None  # new weights: the derived copy is rebuilt on the next decode call
        return super()._load_from_state_dict(*args, **kwargs)

    def tiled_for(self, x):
        """The tiled weight copy when ``x`` is eligible for the tensor-core kernel (row-wise format, fp16, CUDA,
        in_features % 128 == 0; built once per device on first use), else None."""
        if not self.sm7x_rowwise:
            return None
        rows = x.numel() // self.in_features
        if not (rows <= TILED_MAX_ROWS and x.dtype == torch.float16 and x.is_cuda and self.in_features % 128 == 0
                and self.row_scale.dtype == torch.float16):
            return None
        t = self._tiled
        if t is None or t.device != x.device:
            t = self._tiled = w8_repack_tiled(self.q_row)
        return t

    def _lin(self, x, **kw):
        if self.sm7x_rowwise:
            t = self.tiled_for(x)
            if t is not None:
                return w8_tiled_linear_group((x,), (t,), (self.row_scale,), self.out_features, self.in_features, **kw)[0]
            return w8_linear(x, self.q_row, self.row_scale, **kw)
        y = mm8_matmul(x, self.w_u8, self.mx, self.rx, self.my, self.ry)
        if kw.get("relu2"):
            from .prep import relu2_
            y = relu2_(y.contiguous()) if y.numel() % 8 == 0 else torch.relu(y) ** 2
        if kw.get("residual") is not None:
            y = y + kw["residual"].reshape(y.shape)
        if kw.get("out") is not None:
            kw["out"].copy_(y.reshape(kw["out"].shape))
            return kw["out"]
        return y

    def forward(self, x):
        y = self._lin(x)
        return y if self.bias is None else y + self.bias

    def rwkv7_forward_into(self, x, out):
        if self.bias is None:
            return self._lin(x, out=out)
        out.copy_(self.forward(x))
        return out

    def rwkv7_forward_relu2(self, x):
        if self.bias is None:
            return self._lin(x, relu2=True)
        return torch.relu(self.forward(x)) ** 2

    def rwkv7_forward_add(self, x, residual):
        if self.bias is None:
            return self._lin(x, residual=residual)
        return self.forward(x) + residual

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, mm8(fused={self.fused}, sm7x_rowwise={self.sm7x_rowwise})"


class MM4Linear(torch.nn.Module):
    """``nn.Linear`` replacement with int4 group-wise weights (buffers ``packed_group``, ``group_scales``)."""

    def __init__(self, linear, *, fused=True, group_size=128):
        super().__init__()
        self.in_features, self.out_features = int(linear.weight.shape[1]), int(linear.weight.shape[0])
        self.group_size = int(group_size)
        if self.group_size not in {128, 256}:
            raise ValueError("MM4Linear in this package requires group_size 128 or 256")
        if self.in_features % self.group_size:
            raise ValueError("in_features must be divisible by group_size")
        self.groupwise = True
        packed_group, group_scales, packed_inputs = quantize_w4_groupwise(linear.weight.data, group_size=self.group_size)
        self.register_buffer("packed_group", packed_group)
        self.register_buffer("group_scales", group_scales)
        self.group_zeros = None
        self._tiled = None  # tiled copy for the tensor-core decode kernel (derived, not part of the state dict)
        self.packed_inputs = int(packed_inputs)
        self.m_orig = self.out_features
        if linear.bias is not None:
            self.register_buffer("bias", linear.bias.data.clone())
        else:
            self.bias = None
        self.fused = bool(fused)

    def _load_from_state_dict(self, *args, **kwargs):
        self._tiled = None  # new weights: the derived copy is rebuilt on the next decode call
        return super()._load_from_state_dict(*args, **kwargs)

    def tiled_for(self, x):
        """The tiled weight copy when ``x`` is eligible for the tensor-core decode kernel (built once per device,
        on first use), else None."""
        rows = x.numel() // self.in_features
        if not (rows <= TILED_MAX_ROWS and x.dtype == torch.float16 and x.is_cuda and self.in_features % 128 == 0):
            return None
        t = self._tiled
        if t is None or t.device != x.device:
            t = self._tiled = w4_repack_tiled(self.packed_group, self.group_scales, self.in_features,
                                              self.group_size, self.group_zeros)
        return t

    def _lin(self, x, **kw):
        t = self.tiled_for(x)
        if t is not None:
            return w4_tiled_linear(x, t, self.out_features, self.in_features, **kw)
        return w4_groupwise_linear(x, self.packed_group, self.group_scales, self.out_features, self.in_features,
                                   group_size=self.group_size, zeros=self.group_zeros, **kw)

    def forward(self, x):
        y = self._lin(x)
        return y if self.bias is None else y + self.bias

    def rwkv7_forward_into(self, x, out):
        if self.bias is None:
            return self._lin(x, out=out)
        out.copy_(self.forward(x))
        return out

    def rwkv7_forward_relu2(self, x):
        if self.bias is None:
            return self._lin(x, relu2=True)
        return torch.relu(self.forward(x)) ** 2

    def rwkv7_forward_add(self, x, residual):
        if self.bias is None:
            return self._lin(x, residual=residual)
        return self.forward(x) + residual

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, mm4(group_size={self.group_size})"


class A8W8Linear(torch.nn.Module):
    """Inference-only ``nn.Linear`` replacement using dynamic A8 and W8 (buffers ``q_weight_t``, ``weight_scale``)."""

    def __init__(self, linear):
        super().__init__()
        self.in_features = int(linear.in_features)
        self.out_features = int(linear.out_features)
        q_weight_t, weight_scale = quantize_weight_per_channel_int8(linear.weight)
        self.register_buffer("q_weight_t", q_weight_t)
        self.register_buffer("weight_scale", weight_scale)
        if linear.bias is None:
            self.bias = None
        else:
            self.register_buffer("bias", linear.bias.detach().clone())
        self.fused_ffn = True
        self.sm70_rowwise = False

    def forward(self, x):
        return a8w8_linear(x, self.q_weight_t, self.weight_scale, self.bias)

    def rwkv7_forward_into(self, x, out):
        return a8w8_linear(x, self.q_weight_t, self.weight_scale, self.bias, out=out)

    def rwkv7_forward_add(self, x, residual):
        return a8w8_linear(x, self.q_weight_t, self.weight_scale, self.bias, residual=residual)

    def rwkv7_forward_relu2(self, x):
        return a8w8_linear(x, self.q_weight_t, self.weight_scale, self.bias, relu2=True)

    def rwkv7_forward_ffn(self, x, down, residual):
        """up -> relu^2 (fp16 boundary) -> down + residual; returns None when the pairing does not apply."""
        if not isinstance(down, A8W8Linear) or self.out_features != down.in_features:
            return None
        y = a8w8_ffn(x, self, down, residual)
        if y is not None:
            return y
        from .prep import relu2_
        return down.rwkv7_forward_add(relu2_(self.forward(x).contiguous()), residual)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, dynamic_a8w8"


def quantize_model(model, kind: str, *, min_params: int = 8_000_000, group_size: int = 128, skip=("lm_head",)) -> int:
    """Swap eligible ``nn.Linear`` modules in place (role of quantize_model_mm8 / quantize_model_mm4,
    rwkv7_hf/native_quant_mm8.py:631-684, rwkv7_hf/native_quant_mm4.py:761-832).  ``kind`` in
    {"mm8" (fp16i8 affine), "w8" (row-wise int8), "mm4" (int4 group-wise), "a8w8"}; modules with fewer than ``min_params`` weights or whose name is in ``skip`` stay dense."""
    n = 0
    for parent_name, parent in list(model.named_modules()):
        for name, child in list(parent.named_children()):
            full = f"{parent_name}.{name}" if parent_name else name
            if not isinstance(child, torch.nn.Linear) or child.weight.numel() < min_params:
                continue
            if any(full == s or full.endswith("." + s) for s in skip) or ".lora." in full:
                continue  # the rank-R LoRA linears stay dense (they run on the grouped small-GEMM kernel)
            if kind == "mm8":
                new = MM8Linear(child)
            elif kind == "w8":
                new = MM8Linear(child, rowwise=True)
            elif kind == "mm4":
                if child.in_features % group_size:
                    continue
                new = MM4Linear(child, group_size=group_size)
            elif kind == "a8w8":
                if child.in_features % 16 or child.out_features % 8:
                    continue
                new = A8W8Linear(child)
            else:
                raise ValueError(f"unknown quantisation kind {kind!r}")
            setattr(parent, name, new)
            n += 1
    return n
