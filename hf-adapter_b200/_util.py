"""Host-side helpers shared by the operator wrappers."""
from __future__ import annotations

import torch

from . import _lib

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}


def dt_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported activation dtype {t.dtype}") from None


def stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors, what: str) -> None:
    """There is no CPU path in this package: every tensor must live on one CUDA device."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"{what}: tensors must be CUDA tensors (this package has no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"{what}: tensors must be on the same device")


def same_dtype(first, *rest, what: str) -> None:
    for t in rest:
        if t is not None and t.dtype != first.dtype:
            raise ValueError(f"{what}: dtype mismatch ({t.dtype} vs {first.dtype})")


def ptr(t):
    return 0 if t is None else t.data_ptr()


def no_fallback(force_fallback: bool, what: str) -> None:
    if force_fallback:
        raise RuntimeError(f"{what}: force_fallback=True requests the pure-PyTorch path, which this package does not ship")
