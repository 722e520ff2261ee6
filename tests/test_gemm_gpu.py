"""The dense tensor-core GEMM with fused epilogues (rwkv7_gemm) against an fp32 matmul of the same fp16 / bf16
operands: ragged and multi-wave shapes, bias, relu^2 of the rounded value, residual add; the A8W8 linear whose
dequantisation now rides in the same kernel's epilogue stays pinned to the oracle's integer arithmetic elsewhere
(test_quant_gpu.py, test_configs_gpu.py).  Tolerances: fp32 accumulation, one rounding to the activation type."""
import pytest
import torch

import hf_adapter_b200 as hb
from hf_adapter_b200 import _lib

pytestmark = pytest.mark.gpu


def _ref(x, w, bias, relu2, residual):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if relu2:
        y = torch.relu(y.to(x.dtype).float()) ** 2
    elif residual is not None:
        y = y + residual.float()
    return y


@pytest.mark.parametrize("M,K,N", [(64, 128, 256), (130, 1000, 264), (1, 64, 8), (257, 4096, 1000), (4096, 512, 4096),
                                   (300, 16384, 512), (2048, 2560, 10240)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_epilogues(M, K, N, dtype):
    if dtype == torch.bfloat16 and M * N > 1 << 22:
        pytest.skip("the large shapes run once, in fp16")
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(dtype)
    bias = torch.randn(N, device="cuda", generator=g).to(dtype)
    res = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    tol = dict(rtol=2e-3, atol=2e-3) if dtype == torch.float16 else dict(rtol=1.6e-2, atol=1.6e-2)
    for b_, relu2, r_ in ((None, False, None), (bias, False, res), (None, True, None), (bias, True, None), (None, False, res)):
        y = hb.dense_linear(x, w, b_, relu2=relu2, residual=r_)
        assert y.shape == (M, N) and y.dtype == dtype
        # squaring doubles the relative error of a value that rounded one way here and the other way in the reference
        t_ = {k: v * (2.5 if relu2 else 1.0) for k, v in tol.items()}
        torch.testing.assert_close(y.float(), _ref(x, w, b_, relu2, r_), **t_)
    again = hb.dense_linear(x, w, bias, residual=res)
    assert torch.equal(again, hb.dense_linear(x, w, bias, residual=res))  # deterministic
    assert _lib.kernel_status() == 0


def test_gemm_into_views_and_batched_rows():
    x = torch.randn(3, 50, 256, device="cuda", dtype=torch.float16)
    w = torch.randn(384, 256, device="cuda", dtype=torch.float16) / 16
    out = torch.empty(3, 50, 384, device="cuda", dtype=torch.float16)
    y = hb.dense_linear(x, w, out=out)
    assert y.data_ptr() == out.data_ptr() and y.shape == (3, 50, 384)
    torch.testing.assert_close(y.float(), x.float() @ w.float().t(), rtol=2e-3, atol=2e-3)
    with pytest.raises(ValueError):
        hb.dense_linear(x.float(), w.float())
    with pytest.raises(ValueError):
        hb.dense_linear(x, w, relu2=True, residual=out)
    with pytest.raises(ValueError):
        hb.dense_linear(x[..., :100].contiguous(), w[:, :100].contiguous())  # K % 8


def test_fused_sequence_ffn_runs_on_the_library_gemm():
    B, T, D, F_ = 2, 96, 256, 1024
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(B, T, D, device="cuda", generator=g).half()
    prev = torch.randn(B, D, device="cuda", generator=g).half()
    mix = torch.rand(D, device="cuda", generator=g).half()
    wk = (torch.randn(F_, D, device="cuda", generator=g) / 16).half()
    wv = (torch.randn(D, F_, device="cuda", generator=g) / 32).half()
    before = _lib.LAUNCHES
    out, nxt = hb.fused_sequence_ffn(x, prev, mix, wk, wv)
    assert _lib.LAUNCHES - before == 3  # shift-mix, key GEMM with relu^2, value GEMM
    shifted = torch.cat([prev[:, None], x[:, :-1]], 1)
    mixed = (x.float() + (shifted.float() - x.float()) * mix.float()).half()
    mid = (torch.relu((mixed.float() @ wk.float().t()).half().float()) ** 2).half()
    want = mid.float() @ wv.float().t()
    torch.testing.assert_close(out.float(), want, rtol=4e-3, atol=4e-3)
    assert torch.equal(nxt, x[:, -1])


@pytest.mark.parametrize("M,K,N", [(64, 256, 1000), (5, 128, 65536), (200, 512, 4096), (64, 4096, 65536)])
def test_fused_argmax_equals_argmax_of_stored_logits(M, K, N):
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).half()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).half()
    w[N // 2] = w[3]  # two identical columns: a guaranteed tie wherever column 3 wins
    x[0] = 0  # an all-equal row: index 0 must win
    logits = hb.dense_linear(x, w)
    idx, val = hb.dense_argmax(x, w, return_values=True)
    assert idx.dtype == torch.int64 and torch.equal(idx, logits.argmax(-1))
    assert torch.equal(val, logits.float().max(-1).values)
    assert torch.equal(hb.dense_argmax(x, w), idx) and int(idx[0]) == 0
    assert _lib.kernel_status() == 0
