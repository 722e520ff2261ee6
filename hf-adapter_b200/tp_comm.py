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


class PeerRowSum:
    """The sums that the row kernels take in themselves (``rwkv7_tp_ffn_add_norm_mix`` after ``o_proj``,
    ``rwkv7_tp_attn_norm_mix6`` after ``ffn.value``): an inbox ``[2][P][max_rows * width]`` on every rank in which every
    4 bytes of payload sit beside the 4-byte call number (no flag array).  Same rules as ``PeerAllReduce``: one instance per stream, the same sequence of calls on every rank."""

    @staticmethod
    def resident_rows(width: int, dtype) -> int:
        """CTAs (one row at a time each) of the row kernels that are resident at once on the current device: their
        largest grid (0: unsupported width or dtype)."""
        if dtype not in (torch.float16, torch.bfloat16):
            return 0
        return int(_lib.lib.rwkv7_tp_rows_resident(int(width), _lib.F16 if dtype == torch.float16 else _lib.BF16))

    def __init__(self, group, max_rows: int, width: int, device, dtype=torch.float16, wait_ms: int = 2000,
                 max_ctas: int = 0):
        """``max_ctas`` > 0 bounds the grid of the row kernels below what is resident at once: instances whose kernels
        run side by side on two streams pass ``resident_rows(...) // 2`` each."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("PeerRowSum takes fp16 or bf16 rows")
        self.max_ctas = int(max_ctas)
        self.group, self.rank, self.world = group, dist.get_rank(group), dist.get_world_size(group)
        self.width, self.wait_ms, self.dtype = int(width), int(wait_ms), dtype
        self.dtype_code = _lib.F16 if dtype == torch.float16 else _lib.BF16
        self.max_rows = int(max_rows)
        if self.max_rows <= 0 or self.resident_rows(self.width, dtype) <= 0:
            raise ValueError(f"rows of {self.width} values are not supported by the tensor-parallel row kernels")
        self.slot_elems = (self.max_rows * self.width + 7) // 8 * 8
        self.buf = symm_mem.empty(2 * self.world * self.slot_elems * 4, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.buf.zero_()
        self.counters = torch.zeros(2, device=device, dtype=torch.int32)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # nobody pushes before every inbox is zero
        self._inbox_arr = (ctypes.c_void_p * self.world)(*[int(p) for p in self.handle.buffer_ptrs])
        self._inbox = ctypes.cast(self._inbox_arr, _lib.PP)

    def takes(self, partial) -> bool:
        return (partial.is_cuda and partial.dtype == self.dtype and partial.dim() == 2 and partial.is_contiguous()
                and int(partial.shape[1]) == self.width and 0 < int(partial.shape[0]) <= self.max_rows)

    def _check(self, partial, *same):
        if not self.takes(partial):
            raise ValueError(f"PeerRowSum takes contiguous CUDA {self.dtype} [rows <= {self.max_rows}, {self.width}] partials")
        for t in same:
            if t.dtype != self.dtype or not t.is_cuda or not t.is_contiguous():
                raise ValueError("every operand must be a contiguous CUDA tensor of the partial's dtype")

    def ffn_add_norm_mix(self, residual, partial, previous, norm_weight, norm_bias, mix, *, eps: float = 1e-5,
                         slot_ids=None):
        """``fused_ffn_add_norm_mix_decode(residual, sum over ranks of partial, ...)``: returns ``(x, mixed)``."""
        self._check(partial, residual, previous, norm_weight, norm_bias, mix)
        rows = int(partial.shape[0])
        if tuple(residual.shape) != tuple(partial.shape):
            raise ValueError("residual and partial must have identical shapes")
        if slot_ids is None and tuple(previous.shape) != tuple(partial.shape):
            raise ValueError("previous must have the partial's shape (or pass slot_ids)")
        res_out, mixed = torch.empty_like(partial), torch.empty_like(partial)
        _lib.check(_lib.lib.rwkv7_tp_ffn_add_norm_mix(
            ptr(residual), ptr(partial), ptr(previous), ptr(slot_ids), ptr(norm_weight),
            ptr(norm_bias), ptr(mix), ptr(res_out), ptr(mixed), self._inbox, ptr(self.counters), self.rank,
            self.world, rows, self.width, self.slot_elems, self.max_ctas, float(eps), self.wait_ms, self.dtype_code,
            stream_ptr(partial)), "tp_ffn_add_norm_mix")
        return res_out, mixed

    def attn_norm_mix6(self, partial, previous, norm_weight, norm_bias, mixes, *, eps: float = 1e-5, slot_ids=None):
        """``x = sum over ranks of partial``; ``fused_attn_norm_mix6_decode(x, ...)``: returns ``(x, (xr,xw,xk,xv,xa,xg))``."""
        mixes = tuple(mixes)
        if len(mixes) != 6:
            raise ValueError("six mix vectors (r, w, k, v, a, g)")
        self._check(partial, previous, norm_weight, norm_bias, *mixes)
        rows = int(partial.shape[0])
        if slot_ids is None and tuple(previous.shape) != tuple(partial.shape):
            raise ValueError("previous must have the partial's shape (or pass slot_ids)")
        x = torch.empty_like(partial)
        s = torch.empty((6, rows, self.width), device=partial.device, dtype=partial.dtype)
        mixes_p, _k1 = _lib.ptr_array([m.data_ptr() for m in mixes])
        outs_p, _k2 = _lib.ptr_array([s[i].data_ptr() for i in range(6)])
        _lib.check(_lib.lib.rwkv7_tp_attn_norm_mix6(
            ptr(partial), ptr(x), ptr(previous), ptr(slot_ids), ptr(norm_weight),
            ptr(norm_bias), mixes_p, outs_p, self._inbox, ptr(self.counters), self.rank, self.world, rows,
            self.width, self.slot_elems, self.max_ctas, float(eps), self.wait_ms, self.dtype_code, stream_ptr(partial)),
            "tp_attn_norm_mix6")
        return x, tuple(s[i] for i in range(6))


# Communicators live as long as the process.  Their buffers are mapped into every rank of the group; a rank that
# released one while the others still held the mapping (a model deleted on one rank a moment before the others, a
# communicator re-made for a larger batch in the middle of a step) was followed by launch failures on OTHER ranks on
# NVSwitch machines.  So nothing is released before the process ends: whoever creates a communicator for a model hands
# it to keep_alive(), and the ranks leave together (a barrier, then exit).
_KEPT = []


def keep_alive(comm):
    """Hold ``comm`` until the process ends.  The price: every tensor-parallel model made in a process adds its
    communicators' buffers (2 * P * 1024 rows * width * 4 bytes for the row kernels, half of that for the stand-alone
    sum) to what the process holds; a server makes one model per process."""
    _KEPT.append(comm)
    return comm
