"""Dense projections over many rows on this library's tensor-core GEMM (csrc/gemm_umma.cu), with the bias, the
relu^2 of the FFN or the residual add fused into the epilogue.  The role of the reference's ``tl.dot`` GEMMs with
fused epilogues (rwkv7_hf/fused_ffn.py:39-232) and of the ``F.linear`` calls of its layer-wise prefill
(rwkv7_hf/native_jit_prefill.py:964-1040)."""
from __future__ import annotations

import torch

from . import _lib
from ._util import dt_code, ptr, stream_ptr

# below this many rows a projection is a weight-streaming problem (the decode kernels' job), not a GEMM
MIN_ROWS = 64


def takes(x, weight) -> bool:
    """Whether ``dense_linear`` runs ``x @ weight.T``: fp16 / bf16 CUDA operands of one dtype, K a multiple of 8."""
    return (x.is_cuda and weight.is_cuda and x.dtype == weight.dtype and x.dtype in (torch.float16, torch.bfloat16)
            and weight.dim() == 2 and int(weight.shape[1]) % 8 == 0 and int(x.shape[-1]) == int(weight.shape[1]))


def dense_linear(x, weight, bias=None, *, relu2: bool = False, residual=None, out=None):
    """``x [..., K] @ weight[N, K].T (+ bias)`` then ``relu(.)**2`` (of the value rounded to the activation type, as
    ``torch.relu(linear(x)) ** 2`` computes it) or ``+ residual``.  One kernel launch."""
    if not takes(x, weight):
        raise ValueError("dense_linear needs fp16 / bf16 CUDA operands of one dtype with K % 8 == 0")
    if relu2 and residual is not None:
        raise ValueError("the relu^2 epilogue takes no residual")
    N, K = (int(v) for v in weight.shape)
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    w = weight if weight.is_contiguous() else weight.contiguous()
    M = int(x2.shape[0])
    res = None
    if residual is not None:
        res = residual.reshape(M, N)
        if res.dtype != x.dtype:
            raise ValueError("residual must have the activation dtype")
        res = res if res.is_contiguous() else res.contiguous()
    if bias is not None and (bias.dtype != x.dtype or int(bias.numel()) != N):
        raise ValueError("bias must be [out_features] in the activation dtype")
    y = torch.empty((M, N), device=x.device, dtype=x.dtype) if out is None else out.reshape(M, N)
    if not y.is_contiguous() or y.dtype != x.dtype:
        raise ValueError("out must be contiguous and have the activation dtype")
    _lib.check(_lib.lib.rwkv7_gemm(ptr(x2), ptr(w), ptr(bias), ptr(res), ptr(y), M, K, N, 1 if relu2 else 0, dt_code(x2),
                                   stream_ptr(x2)), "gemm")
    return y.reshape(*x.shape[:-1], N)


def dense_argmax(x, weight, *, return_values: bool = False):
    """``argmax(x @ weight.T, dim=-1)`` per row without materialising the logits: the GEMM's epilogue keeps the best
    column of every tile and a small second kernel folds the tiles.  Equal to ``torch.argmax`` of the fp16 / bf16
    logits (values are rounded to that type before they are compared; the lowest index wins a tie).  With
    ``return_values`` also the winning logit per row (fp32), which a vocabulary-sharded head exchanges."""
    if not takes(x, weight):
        raise ValueError("dense_argmax needs fp16 / bf16 CUDA operands of one dtype with K % 8 == 0")
    N, K = (int(v) for v in weight.shape)
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    w = weight if weight.is_contiguous() else weight.contiguous()
    M = int(x2.shape[0])
    nbytes = int(_lib.lib.rwkv7_gemm_argmax_workspace_bytes(M, N))
    ws = torch.empty((nbytes,), device=x.device, dtype=torch.uint8)
    idx = torch.empty((M,), device=x.device, dtype=torch.int64)
    val = torch.empty((M,), device=x.device, dtype=torch.float32) if return_values else None
    _lib.check(_lib.lib.rwkv7_gemm_argmax(ptr(x2), ptr(w), ptr(ws), nbytes, ptr(val), ptr(idx), M, K, N, dt_code(x2),
                                          stream_ptr(x2)), "gemm_argmax", kernels=2)
    idx = idx.reshape(x.shape[:-1])
    return (idx, val.reshape(x.shape[:-1])) if return_values else idx
