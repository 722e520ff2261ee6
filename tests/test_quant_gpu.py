"""GPU parity of the quantised projections: bit-exact integer work (activation quantiser, int8 GEMM
accumulators), reference-format GEMV/GEMM outputs against the golden fixtures and the oracle."""
import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from oracle import rwkv7_oracle as O
from tests.gpu_util import cu, golden, npf

pytestmark = pytest.mark.gpu


def test_formats_against_golden():
    g = golden("quant.npz")
    x = cu(g["x"])
    y = hb.w8_linear(x, cu(g["w8_q"]), cu(g["w8_s"]))
    np.testing.assert_allclose(npf(y), g["w8_y"].astype(np.float32), rtol=2e-3, atol=2e-3)
    y = hb.w4_groupwise_linear(x, cu(g["w4g_packed"]), cu(g["w4g_scales"]), 96, 256, group_size=128)
    np.testing.assert_allclose(npf(y), g["w4g_y"].astype(np.float32), rtol=2e-3, atol=2e-3)
    y = hb.a8w8_linear(x, cu(g["a8w8_q_t"]), cu(g["a8w8_s"]))
    ref = g["a8w8_y"].astype(np.float64).ravel()
    mine = npf(y).astype(np.float64).ravel()
    assert mine @ ref / np.linalg.norm(mine) / np.linalg.norm(ref) >= 0.9999  # the reference's own gate
    yo = O.a8w8_linear(g["x"], g["a8w8_q_t"], g["a8w8_s"])[0]
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("rows,K", [(1, 8), (5, 256), (64, 4096), (3, 16384)])
def test_a8_quantiser_bit_exact(rows, K):
    rng = np.random.default_rng(K)
    x = rng.standard_normal((rows, K)).astype(np.float16)
    x[0, :4] = [0.5, -0.5, 1.5, -2.5]  # ties
    if rows > 2:
        x[2] = 0  # all-zero row -> scale floor 1e-5
    qo, so = O.dynamic_a8_quant(x)
    q, s = hb.dynamic_a8_quant(cu(x))
    assert np.array_equal(s.cpu().numpy(), so)
    assert np.array_equal(q.cpu().numpy(), qo)


@pytest.mark.parametrize("M,K,Nn", [(1, 16, 8), (17, 64, 24), (64, 256, 96), (130, 4096, 136), (256, 512, 256), (384, 1024, 512)])
def test_int8_gemm_bit_exact(M, K, Nn):
    rng = np.random.default_rng(M * 7 + Nn)
    qa = rng.integers(-127, 128, (M, K), dtype=np.int8)
    qw = rng.integers(-127, 128, (Nn, K), dtype=np.int8)
    acc = hb.int8_mm(cu(qa), cu(qw))
    assert np.array_equal(acc.cpu().numpy(), O.int8_gemm_i32(qa, qw.T))


def test_int8_gemm_extreme_values():
    M, K, Nn = 128, 4096, 128
    qa = np.full((M, K), -127, np.int8)
    qw = np.full((Nn, K), 127, np.int8)
    qw[::2] = -127
    acc = hb.int8_mm(cu(qa), cu(qw))
    assert np.array_equal(acc.cpu().numpy(), O.int8_gemm_i32(qa, qw.T))


@pytest.mark.parametrize("M", [1, 2, 3, 8, 17, 64])
@pytest.mark.parametrize("K,Nn", [(256, 40), (1024, 264)])
def test_w4g_w8_gemv_against_oracle(M, K, Nn):
    rng = np.random.default_rng(M + K)
    W = (0.02 * rng.standard_normal((Nn, K))).astype(np.float16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    res = rng.standard_normal((M, Nn)).astype(np.float16)
    packed, scales = O.quantize_w4_groupwise(W, 128)
    yo = O.w4_groupwise_linear(x, packed, scales)
    y = hb.w4_groupwise_linear(cu(x), cu(packed), cu(scales), Nn, K, group_size=128)
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=2e-3, atol=2e-3)
    yr = hb.w4_groupwise_linear(cu(x), cu(packed), cu(scales), Nn, K, relu2=True)
    ro = np.maximum(yo.astype(np.float32), 0) ** 2
    np.testing.assert_allclose(npf(yr), ro.astype(np.float16).astype(np.float32), rtol=4e-3, atol=4e-3)
    ya = hb.w4_groupwise_linear(cu(x), cu(packed), cu(scales), Nn, K, residual=cu(res))
    np.testing.assert_allclose(npf(ya), (yo.astype(np.float32) + res.astype(np.float32)), rtol=2e-3, atol=4e-3)
    # explicit zero-points: zeros == 8 reproduces the implicit format bit for bit; random zeros follow the oracle
    z8 = np.full(scales.shape, 8, np.uint8)
    assert torch.equal(hb.w4_groupwise_linear(cu(x), cu(packed), cu(scales), Nn, K, zeros=cu(z8)), y)
    zr = rng.integers(5, 12, scales.shape, dtype=np.uint8)
    yz = hb.w4_groupwise_linear(cu(x), cu(packed), cu(scales), Nn, K, zeros=cu(zr))
    np.testing.assert_allclose(npf(yz), O.w4_groupwise_linear(x, packed, scales, zr).astype(np.float32), rtol=2e-3, atol=3e-3)
    # dequantised weight is bit-exact
    Wd = hb.w4_dequant(cu(packed), cu(scales), K, 128)
    assert np.array_equal(Wd.cpu().numpy(), O.dequant_w4_groupwise(packed, scales))
    q, s = O.quantize_w8_row(W)
    y8 = hb.w8_linear(cu(x), cu(q), cu(s))
    np.testing.assert_allclose(npf(y8), O.w8_linear(x, q, s).astype(np.float32), rtol=2e-3, atol=2e-3)


def test_many_rows_take_the_gemm_route():
    rng = np.random.default_rng(9)
    K, Nn, M = 512, 128, 200
    W = (0.02 * rng.standard_normal((Nn, K))).astype(np.float16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    packed, scales = O.quantize_w4_groupwise(W, 128)
    y = hb.w4_groupwise_linear(cu(x), cu(packed), cu(scales), Nn, K)
    np.testing.assert_allclose(npf(y), O.w4_groupwise_linear(x, packed, scales).astype(np.float32), rtol=2e-3, atol=2e-3)
    q, s = O.quantize_w8_row(W)
    np.testing.assert_allclose(npf(hb.w8_linear(cu(x), cu(q), cu(s))), O.w8_linear(x, q, s).astype(np.float32), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("M", [1, 17, 300])
def test_a8w8_linear_against_oracle(M):
    rng = np.random.default_rng(M)
    K, Nn = 512, 264
    W = (0.02 * rng.standard_normal((Nn, K))).astype(np.float16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    bias = (0.1 * rng.standard_normal(Nn)).astype(np.float16)
    res = rng.standard_normal((M, Nn)).astype(np.float16)
    qt, st = O.quantize_weight_per_channel_int8(W)
    yo, acc, qa, sa = O.a8w8_linear(x, qt, st, bias, res)
    lin = torch.nn.Linear(K, Nn, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(W.astype(np.float32)))
        lin.bias.copy_(torch.from_numpy(bias.astype(np.float32)))
    mod = hb.A8W8Linear(lin.half()).cuda()
    assert np.array_equal(mod.q_weight_t.cpu().numpy(), qt) and np.array_equal(mod.weight_scale.cpu().numpy(), st)
    y = mod.rwkv7_forward_add(cu(x), cu(res))
    np.testing.assert_allclose(npf(y), yo.astype(np.float32), rtol=1e-3, atol=2e-3)
    # the pieces: integer accumulators bit-exact
    q_gpu, s_gpu = hb.dynamic_a8_quant(cu(x))
    assert np.array_equal(q_gpu.cpu().numpy(), qa)
    assert np.array_equal(hb.int8_mm(q_gpu, mod.q_weight_t.t()).cpu().numpy(), acc)


@pytest.mark.parametrize("M,K,Nn", [(1, 128, 8), (5, 512, 128), (16, 1024, 200), (33, 2048, 384), (64, 4096, 512), (64, 16384, 256),
                                    (64, 4096, 4096), (130, 1024, 256), (256, 4096, 512),
                                    # long K ranges per CTA with 128 rows per pass: every ring of that variant wraps
                                    (128, 2048, 8192), (192, 4096, 4096),
                                    # the per-rank shards of an 8-way head-sharded run at batch 512: r/k/v, o, key, value
                                    (512, 4096, 512), (512, 512, 4096), (512, 4096, 2048), (512, 2048, 4096)])
def test_w4g_tensor_core_path(M, K, Nn):
    """tcgen05 kernel on the tiled weight copy (fp16, K % 128 == 0, 1..64 rows, any Nout): all epilogues, zero-points,
    group 256, determinism, and no bounded wait ever giving up."""
    from hf_adapter_b200 import _lib
    rng = np.random.default_rng(M + K + Nn)
    W = (0.02 * rng.standard_normal((Nn, K))).astype(np.float16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    res = rng.standard_normal((M, Nn)).astype(np.float16)
    packed, scales = O.quantize_w4_groupwise(W, 128)
    yo = O.w4_groupwise_linear(x, packed, scales).astype(np.float32)
    xg, pg, sg = cu(x), cu(packed), cu(scales)
    _lib.kernel_status(True)
    tiled = hb.w4_repack_tiled(pg, sg, K, 128)
    y = hb.w4_tiled_linear(xg, tiled, Nn, K)
    assert _lib.kernel_status(True) == 0
    tol_abs = 2e-3 * max(1.0, float(np.abs(yo).max()))
    np.testing.assert_allclose(npf(y), yo, rtol=2e-3, atol=tol_abs)
    assert torch.equal(hb.w4_tiled_linear(xg, tiled, Nn, K), y)  # deterministic split-K
    yr = hb.w4_tiled_linear(xg, tiled, Nn, K, relu2=True)
    ro = (np.maximum(yo.astype(np.float16).astype(np.float32), 0) ** 2).astype(np.float16).astype(np.float32)
    np.testing.assert_allclose(npf(yr), ro, rtol=6e-3, atol=tol_abs * 4)
    ya = hb.w4_tiled_linear(xg, tiled, Nn, K, residual=cu(res))
    np.testing.assert_allclose(npf(ya), yo + res.astype(np.float32), rtol=2e-3, atol=tol_abs * 2)
    zr = rng.integers(5, 12, scales.shape, dtype=np.uint8)
    yz = hb.w4_tiled_linear(xg, hb.w4_repack_tiled(pg, sg, K, 128, zeros=cu(zr)), Nn, K)
    zo = O.w4_groupwise_linear(x, packed, scales, zr).astype(np.float32)
    np.testing.assert_allclose(npf(yz), zo, rtol=2e-3, atol=2e-3 * max(1.0, float(np.abs(zo).max())))
    if K % 256 == 0:
        p2, s2 = O.quantize_w4_groupwise(W, 256)
        y2 = hb.w4_tiled_linear(xg, hb.w4_repack_tiled(cu(p2), cu(s2), K, 256), Nn, K)
        np.testing.assert_allclose(npf(y2), O.w4_groupwise_linear(x, p2, s2, None, 256).astype(np.float32), rtol=2e-3, atol=tol_abs)
    # the module routes decode-size inputs through the same kernel
    lin = torch.nn.Linear(K, Nn, bias=False)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(W.astype(np.float32)))
    mod = hb.MM4Linear(lin.half(), group_size=128).cuda()
    assert torch.equal(mod(xg), y) and mod._tiled is not None
    assert _lib.kernel_status(True) == 0


@pytest.mark.parametrize("G,M,K,Nn", [(3, 64, 4096, 4096), (3, 7, 512, 200), (2, 130, 1024, 256), (4, 64, 1024, 128), (1, 33, 2048, 384)])
def test_w4g_grouped_projections(G, M, K, Nn):
    """G projections of one shape in a single launch: each output equals the oracle (and, where the split-K plan is
    the same, the single-projection launch bit for bit); relu^2 epilogue; wrong group sizes are refused."""
    from hf_adapter_b200 import _lib
    rng = np.random.default_rng(G * 1000 + M + K + Nn)
    xs, tiled, ref = [], [], []
    for g in range(G):
        W = (0.02 * rng.standard_normal((Nn, K))).astype(np.float16)
        x = rng.standard_normal((M, K)).astype(np.float16)
        packed, scales = O.quantize_w4_groupwise(W, 128)
        ref.append(O.w4_groupwise_linear(x, packed, scales).astype(np.float32))
        xs.append(cu(x))
        tiled.append(hb.w4_repack_tiled(cu(packed), cu(scales), K, 128))
    _lib.kernel_status(True)
    ys = hb.w4_tiled_linear_group(xs, tiled, Nn, K)
    assert _lib.kernel_status(True) == 0 and len(ys) == G
    for y, yo, x, t in zip(ys, ref, xs, tiled):
        tol_abs = 2e-3 * max(1.0, float(np.abs(yo).max()))
        np.testing.assert_allclose(npf(y), yo, rtol=2e-3, atol=tol_abs)
        np.testing.assert_allclose(npf(y), npf(hb.w4_tiled_linear(x, t, Nn, K)), rtol=2e-3, atol=tol_abs)
    again = hb.w4_tiled_linear_group(xs, tiled, Nn, K)
    assert all(torch.equal(a, b) for a, b in zip(again, ys))
    yr = hb.w4_tiled_linear_group(xs, tiled, Nn, K, relu2=True)
    for y, yo in zip(yr, ref):
        ro = (np.maximum(yo.astype(np.float16).astype(np.float32), 0) ** 2).astype(np.float16).astype(np.float32)
        np.testing.assert_allclose(npf(y), ro, rtol=6e-3, atol=8e-3 * max(1.0, float(np.abs(yo).max())))
    with pytest.raises(ValueError):
        hb.w4_tiled_linear_group(xs * 5, tiled * 5, Nn, K)


@pytest.mark.parametrize("G,M,K,Nn", [(1, 1, 128, 8), (1, 5, 512, 200), (3, 64, 2560, 2560), (1, 64, 10240, 2560), (1, 64, 2560, 10240),
                                      (1, 130, 1024, 256), (2, 512, 1024, 384), (1, 64, 4096, 16384)])
def test_w8_tensor_core_path(G, M, K, Nn):
    """int8 per-output-channel weights on the tcgen05 kernel (tiled copy, exact integer weights in the MMA, channel
    scale on the fp32 accumulator) against the oracle's w8_linear (materialised fp16 weight): all epilogues, grouped
    launches, determinism, the module route, and no bounded wait giving up."""
    from hf_adapter_b200 import _lib
    rng = np.random.default_rng(G * 31 + M + K + Nn)
    xs, tiled, scales, ref = [], [], [], []
    for g in range(G):
        W = (0.02 * rng.standard_normal((Nn, K))).astype(np.float16)
        x = rng.standard_normal((M, K)).astype(np.float16)
        q, s = O.quantize_w8_row(W)
        ref.append(O.w8_linear(x, q, s, hi=True).astype(np.float32))
        xs.append(cu(x)); scales.append(cu(s)); tiled.append(hb.w8_repack_tiled(cu(q)))
    _lib.kernel_status(True)
    ys = hb.w8_tiled_linear_group(xs, tiled, scales, Nn, K)
    assert _lib.kernel_status(True) == 0 and len(ys) == G
    for y, yo in zip(ys, ref):
        tol_abs = 2e-3 * max(1.0, float(np.abs(yo).max()))
        np.testing.assert_allclose(npf(y), yo, rtol=2e-3, atol=tol_abs)
    again = hb.w8_tiled_linear_group(xs, tiled, scales, Nn, K)
    assert all(torch.equal(a, b) for a, b in zip(again, ys))
    yr = hb.w8_tiled_linear_group(xs, tiled, scales, Nn, K, relu2=True)
    for y, yo in zip(yr, ref):
        ro = (np.maximum(yo.astype(np.float16).astype(np.float32), 0) ** 2).astype(np.float16).astype(np.float32)
        np.testing.assert_allclose(npf(y), ro, rtol=6e-3, atol=8e-3 * max(1.0, float(np.abs(yo).max())))
    res = rng.standard_normal((M, Nn)).astype(np.float16)
    (ya,) = hb.w8_tiled_linear_group(xs[:1], tiled[:1], scales[:1], Nn, K, residual=cu(res))
    np.testing.assert_allclose(npf(ya), ref[0] + res.astype(np.float32), rtol=2e-3, atol=4e-3 * max(1.0, float(np.abs(ref[0]).max())))
    if K % 128 == 0 and M <= 512:
        lin = torch.nn.Linear(K, Nn, bias=False)
        with torch.no_grad():
            lin.weight.copy_(torch.from_numpy((0.02 * rng.standard_normal((Nn, K))).astype(np.float32)))
        mod = hb.MM8Linear(lin.half(), rowwise=True).cuda()
        y_mod = mod(xs[0])
        assert mod._tiled is not None
        yo = O.w8_linear(npf(xs[0]).astype(np.float16), mod.q_row.cpu().numpy(), mod.row_scale.cpu().numpy(), hi=True).astype(np.float32)
        np.testing.assert_allclose(npf(y_mod), yo, rtol=2e-3, atol=2e-3 * max(1.0, float(np.abs(yo).max())))
        # new weights through load_state_dict drop the derived tiled copy
        sd = {k_: v_.clone() for k_, v_ in mod.state_dict().items()}
        sd["q_row"] = -sd["q_row"]
        mod.load_state_dict(sd)
        assert mod._tiled is None
        np.testing.assert_allclose(npf(mod(xs[0])), -yo, rtol=2e-3, atol=2e-3 * max(1.0, float(np.abs(yo).max())))
    assert _lib.kernel_status(True) == 0


@pytest.mark.parametrize("M", [5, 64, 300])
def test_a8w8_relu2_epilogue(M):
    """relu^2 in the A8W8 linear's epilogue == relu(a8w8_linear(x))**2 computed on the stored fp16 output, on the
    mma.sync route (M < 64) and on the tensor-core route with the fused dequantisation."""
    torch.manual_seed(M)
    K, Nn = 512, 264
    lin = torch.nn.Linear(K, Nn, bias=True).half()
    mod = hb.A8W8Linear(lin).cuda()
    x = torch.randn(M, K, device="cuda", dtype=torch.float16)
    plain = mod(x)
    want = (torch.relu(plain.float()) ** 2).half()
    got = mod.rwkv7_forward_relu2(x)
    assert torch.equal(got, want)
    with pytest.raises(ValueError):
        hb.a8w8_linear(x, mod.q_weight_t, mod.weight_scale, relu2=True, residual=plain)
