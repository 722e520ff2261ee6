"""Tensor-parallel sum of ``[rows, D]`` fp16 partial outputs over peer-mapped memory (``rwkv7_tp_allreduce``).

PyTorch supplies the plumbing only: ``torch.distributed._symmetric_memory`` allocates a buffer on every rank and maps
all of them into every process; the kernel of this library then moves the data itself with plain peer stores and flags.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._util import ptr, stream_ptr


class PeerAllReduce:
    """One communicator: an inbox and a flag array on every rank of ``group``.  ``all_reduce`` calls on one instance must
    not overlap on the GPU (use one instance per stream) and every rank must issue the same sequence of calls."""

    def __init__(self, group, max_rows: int, width: int, device, wait_ms: int = 2000):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.group, self.rank, self.world = group, dist.get_rank(group), dist.get_world_size(group)
        self.width, self.wait_ms = int(width), int(wait_ms)
        self.slot_elems = (int(max_rows) * self.width + 7) // 8 * 8
        self.max_ctas = int(_lib.lib.rwkv7_tp_allreduce_max_ctas())
        inbox_bytes = 2 * self.world * self.slot_elems * 2
        flag_bytes = 2 * self.world * self.max_ctas * 4
        self._inbox_bytes = (inbox_bytes + 255) // 256 * 256
        self.buf = symm_mem.empty(self._inbox_bytes + flag_bytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.buf.zero_()
        self.counters = torch.zeros(2, device=device, dtype=torch.int32)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # nobody pushes before every inbox and flag array is zero
        bases = [int(p) for p in self.handle.buffer_ptrs]
        self._inbox = (ctypes.c_void_p * self.world)(*bases)
        self._flags = (ctypes.c_void_p * self.world)(*[b + self._inbox_bytes for b in bases])

    def all_reduce(self, partial, out=None):
        """``out = sum over ranks of partial`` (``out`` may be ``partial`` itself)."""
        if partial.dtype != torch.float16 or not partial.is_cuda or not partial.is_contiguous():
            raise ValueError("PeerAllReduce takes contiguous CUDA fp16 tensors")
        rows = partial.numel() // self.width
        if rows * self.width != partial.numel() or int(partial.shape[-1]) != self.width:
            raise ValueError(f"the last dimension must be {self.width}")
        if out is None:
            out = torch.empty_like(partial)
        _lib.check(_lib.lib.rwkv7_tp_allreduce(ptr(partial), ptr(out), ctypes.cast(self._inbox, _lib.PP),
                                               ctypes.cast(self._flags, _lib.PP), ptr(self.counters), self.rank,
                                               self.world, rows, self.width, self.slot_elems, self.wait_ms, _lib.F16,
                                               stream_ptr(partial)), "tp_allreduce")
        return out
