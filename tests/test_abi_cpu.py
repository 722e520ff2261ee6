"""CPU checks of the boundary: the library loads, exports every symbol the header declares, rejects
bad arguments with the documented codes (no kernel is launched), and the host-side mirror raises the
reference's exception types."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import hf_adapter_b200 as hb
from hf_adapter_b200 import _lib
from oracle import rwkv7_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "rwkv7_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rwkv7_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    syms = header_symbols()
    assert len(syms) >= 20
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/rwkv7_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == syms, "the ctypes table must list exactly the header's symbols"
    assert lib.rwkv7_abi_version() == 1


def test_argument_validation_without_gpu():
    L = _lib.lib
    # null pointers / bad head size / bad epilogue are rejected before any launch
    assert L.rwkv7_wkv7_update(0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 64, 0, 0, 0) == _lib.ERR_INVALID
    assert L.rwkv7_wkv7_update(16, 16, 16, 16, 16, 16, 16, 16, 16, 1, 1, 32, 0, 0, 0) == _lib.ERR_UNSUPPORTED
    assert "head size" in _lib.last_error()
    assert L.rwkv7_wkv7_update(16, 16, 16, 16, 16, 16, 16, 24, 16, 1, 1, 64, 0, 0, 0) == _lib.ERR_ALIGN
    assert L.rwkv7_wkv7_scan(16, 16, 16, 16, 16, 16, 16, 16, 16, 0, 0, 0, 0, 0.0, 1, 4, 1, 64, 0, 7, 0) == _lib.ERR_INVALID
    assert L.rwkv7_w4g_gemv(16, 16, 16, 0, 0, 16, 1, 100, 8, 128, 0, 0, 0) == _lib.ERR_UNSUPPORTED
    assert L.rwkv7_w4g_gemv(16, 16, 16, 0, 0, 16, 1, 128, 8, 128, 2, 0, 0) == _lib.ERR_INVALID  # add without residual
    assert L.rwkv7_a8w8_linear(16, 16, 16, 0, 0, 16, 256, 8, 4, 64, 64, 0, 0) == _lib.ERR_WORKSPACE
    assert L.rwkv7_layer_norm(16, 16, 16, 16, 1, 12, 1e-5, 0, 0) == _lib.ERR_UNSUPPORTED
    assert L.rwkv7_a8w8_workspace_bytes(4, 64, 64) >= 4 * 64 + 4 * 4 + 4 * 64 * 4
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_UNSUPPORTED, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.ERR_CUDA, "x")


def test_no_cpu_fallback():
    r = torch.zeros(1, 1, 64)
    s = torch.zeros(1, 1, 64, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        hb.fused_recurrent_update(r, r, r, r, r, r, s)
    with pytest.raises(RuntimeError, match="force_fallback"):
        hb.fused_recurrent_update(r, r, r, r, r, r, s, force_fallback=True)
    with pytest.raises(RuntimeError, match="CUDA"):
        hb.w4_groupwise_linear(torch.zeros(1, 128, dtype=torch.float16), torch.zeros(8, 64, dtype=torch.uint8),
                               torch.zeros(8, 1, dtype=torch.float16), 8, 128)


def test_shape_errors_match_reference_types():
    s = torch.zeros(2, 2, 64, 64)
    with pytest.raises(ValueError, match="state must be shaped"):
        hb.fused_recurrent_update(*[torch.zeros(2, 2, 64)] * 6, torch.zeros(2, 64, 64))
    with pytest.raises(ValueError, match=r"r must be shaped"):
        hb.fused_recurrent_update(torch.zeros(2, 3, 64), *[torch.zeros(2, 2, 64)] * 5, s)
    with pytest.raises(ValueError, match="identical shapes"):
        hb.fused_attn_norm_mix6_decode(torch.zeros(2, 8), torch.zeros(3, 8), *[torch.zeros(8)] * 8)
    with pytest.raises(ValueError, match="w_out_dtype"):
        hb.fused_prefill_state_prep(*[torch.zeros(1, 128)] * 4, torch.zeros(128), torch.zeros(128), num_heads=2,
                                    head_dim=64, w_out_dtype="bf16")
    with pytest.raises(ValueError, match="group_size"):
        hb.w4_groupwise_linear(torch.zeros(1, 128), torch.zeros(8, 64, dtype=torch.uint8), torch.zeros(8, 1), 8, 128, group_size=64)


def test_host_quantisers_match_oracle():
    g = torch.Generator().manual_seed(3)
    W = (0.02 * torch.randn(64, 256, generator=g)).half()
    q, s = hb.quantize_w8_row(W)
    qo, so = O.quantize_w8_row(W.numpy())
    assert np.array_equal(q.numpy(), qo) and np.array_equal(s.numpy(), so)
    p, sc, k = hb.quantize_w4_groupwise(W, 128)
    po, sco = O.quantize_w4_groupwise(W.numpy(), 128)
    assert k == 256 and np.array_equal(p.numpy(), po) and np.array_equal(sc.numpy(), sco)
    qt, st = hb.quantize_weight_per_channel_int8(W)
    qto, sto = O.quantize_weight_per_channel_int8(W.numpy())
    assert tuple(qt.shape) == (256, 64) and np.array_equal(qt.numpy(), qto) and np.array_equal(st.numpy(), sto)
    assert qt.t().is_contiguous()  # K-major storage behind the reference-shaped [in,out] buffer


def test_quant_modules_keep_reference_buffer_names():
    lin = torch.nn.Linear(256, 64, bias=False)
    assert set(dict(hb.MM4Linear(lin, group_size=128).named_buffers())) == {"packed_group", "group_scales"}
    mm8 = hb.MM8Linear(lin.half())
    assert set(dict(mm8.named_buffers())) == {"w_u8", "mx", "rx", "my", "ry"}  # the reference's format off sm7x
    assert tuple(mm8.w_u8.shape) == (256, 64) and tuple(mm8.my.shape) == (256, 1) and tuple(mm8.rx.shape) == (64,)
    Wt = lin.weight.data.t().contiguous()
    u8, mx, rx, my, ry = O.quantize_mm8(Wt.float().numpy())
    assert np.array_equal(mm8.w_u8.numpy(), u8) and np.array_equal(mm8.rx.numpy(), rx.astype(np.float16))
    p4, mx4, rx4, my4, ry4, m, mp = hb.quantize_mm4(Wt[:, :63].contiguous())
    po, mxo, rxo, myo, ryo, mo, mpo = O.quantize_mm4(Wt[:, :63].numpy())
    assert (m, mp) == (63, 64) == (mo, mpo) and np.array_equal(p4.numpy(), po) and np.array_equal(ry4.numpy(), ryo)
    assert set(dict(hb.MM8Linear(lin, rowwise=True).named_buffers())) == {"q_row", "row_scale"}  # its sm7x format
    assert set(dict(hb.A8W8Linear(lin).named_buffers())) == {"q_weight_t", "weight_scale"}
    m = torch.nn.Sequential(torch.nn.Linear(256, 64), torch.nn.Linear(64, 8))
    assert hb.quantize_model(m, "mm4", min_params=1000) == 1 and isinstance(m[0], hb.MM4Linear)


def test_cache_contract():
    c = hb.NativeRWKV7Cache.allocate(2, 3, 16, 2, 64, "cpu", torch.float16)
    state, xpa, xpf, v_first = c
    assert len(state) == 2 and state[0].shape == (3, 2, 64, 64) and state[0].dtype == torch.float32
    assert xpa[0].shape == (3, 16) and v_first.shape == (3, 128) and c.get_seq_length() == 0
    state[0][1] += 1
    c._seen_tokens = 5
    d = c.clone()
    d._state[0].zero_()
    assert c._state[0][1].sum() > 0
    c.select_batch(torch.tensor([1, 1]))
    assert c.get_batch_size() == 2 and float(c._state[0][0, 0, 0, 0]) == 1.0
    c.batch_repeat_interleave(2)
    assert c.get_batch_size() == 4
    with pytest.raises(ValueError):
        c.crop(3)
    assert c.crop(9) is c and c.get_seq_length() == 5
    c.crop(0)
    assert c.get_seq_length() == 0 and float(c._state[0].abs().sum()) == 0.0
    assert not c.has_previous_state()


def test_model_state_dict_names_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "model_tiny.npz"))
    ref_names = {k[len("param::"):] for k in g.files if k.startswith("param::")}
    cfg = hb.NativeRWKV7Config(vocab_size=256, hidden_size=128, num_hidden_layers=2, num_heads=2, head_dim=64,
                               intermediate_size=256, decay_low_rank_dim=16, a_low_rank_dim=16, v_low_rank_dim=8,
                               gate_low_rank_dim=32)
    model = hb.RWKV7ForCausalLM(cfg)
    assert set(model.state_dict()) == ref_names
    for k, v in model.state_dict().items():
        assert tuple(v.shape) == tuple(g["param::" + k].shape), k
