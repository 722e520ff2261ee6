"""The allocation-free A8W8 entry point (rwkv7_a8w8_linear_static), for callers that may not allocate device
memory at call time -- a server whose own pool owns all GPU memory, a thread barred from the CUDA allocator.  It
must give exactly what rwkv7_a8w8_linear gives with a caller-provided workspace (same kernels, so bit-identical),
also on a second call that reuses the library's built-in scratch array, and must refuse sizes beyond that array.
Collected last on purpose: a failure here cannot hide the result of any other test."""
import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from hf_adapter_b200 import _lib

pytestmark = pytest.mark.gpu


def _static_call(x, q_row, scale, bias, residual):
    M, K = (int(v) for v in x.shape)
    Nout = int(q_row.shape[0])
    out = torch.empty((M, Nout), device=x.device, dtype=x.dtype)
    ptr = lambda t: 0 if t is None else t.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    code = _lib.lib.rwkv7_a8w8_linear_static(ptr(x), ptr(q_row), ptr(scale), ptr(bias), ptr(residual), ptr(out), M, K, Nout,
                                             _lib.F16, st)
    return code, out


def test_static_scratch_entry_matches_workspace_entry_twice():
    torch.manual_seed(5)
    K, Nout = 512, 264
    W = (0.02 * torch.randn(Nout, K)).half()
    q_t, scale = hb.quantize_weight_per_channel_int8(W)
    q_t, scale = q_t.cuda(), scale.cuda()
    q_row = q_t.t()
    assert q_row.is_contiguous()
    bias = (0.1 * torch.randn(Nout)).half().cuda()
    for call, M in enumerate((37, 5)):  # second call is smaller: stale scratch from the first must not leak in
        x = torch.randn(M, K, device="cuda", dtype=torch.float16)
        res = torch.randn(M, Nout, device="cuda", dtype=torch.float16)
        want = hb.a8w8_linear(x, q_t, scale, bias, residual=res)
        code, got = _static_call(x, q_row, scale, bias, res)
        assert code == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: max diff {(got.float() - want.float()).abs().max().item()}"
        code, got2 = _static_call(x, q_row, scale, None, None)
        assert code == 0 and torch.equal(got2, hb.a8w8_linear(x, q_t, scale))


def test_static_scratch_entry_on_the_tensor_core_path():
    """130 rows x K=1024 takes the tcgen05 int8 GEMM (more than one 128-row tile, a ragged second one) and an
    accumulator region that starts at a rounded-up offset inside the built-in array; 264 outputs leave a ragged
    column tile.  Same kernels as the workspace entry, so bit-identical."""
    torch.manual_seed(6)
    M, K, Nout = 130, 1024, 264
    W = (0.02 * torch.randn(Nout, K)).half()
    q_t, scale = hb.quantize_weight_per_channel_int8(W)
    q_t, scale = q_t.cuda(), scale.cuda()
    q_row = q_t.t()
    assert q_row.is_contiguous()
    assert int(_lib.lib.rwkv7_a8w8_workspace_bytes(M, K, Nout)) <= int(_lib.lib.rwkv7_a8w8_static_capacity_bytes())
    bias = (0.1 * torch.randn(Nout)).half().cuda()
    x = torch.randn(M, K, device="cuda", dtype=torch.float16)
    res = torch.randn(M, Nout, device="cuda", dtype=torch.float16)
    want = hb.a8w8_linear(x, q_t, scale, bias, residual=res)
    for call in range(2):
        code, got = _static_call(x, q_row, scale, bias, res)
        assert code == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: max diff {(got.float() - want.float()).abs().max().item()}"
    assert _lib.lib.rwkv7_kernel_status(0) == 0


def test_static_scratch_entry_rejects_oversize():
    cap = int(_lib.lib.rwkv7_a8w8_static_capacity_bytes())
    assert cap == 8 << 20
    M, K, Nout = 1024, 4096, 4096  # needs 4 MiB + 16 MiB
    assert int(_lib.lib.rwkv7_a8w8_workspace_bytes(M, K, Nout)) > cap
    code = _lib.lib.rwkv7_a8w8_linear_static(256, 256, 256, 0, 0, 256, M, K, Nout, _lib.F16, 0)  # rejected before any pointer is used
    assert code == _lib.ERR_WORKSPACE and "built-in array" in _lib.last_error()
