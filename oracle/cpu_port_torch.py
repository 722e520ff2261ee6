"""Multi-threaded CPU port (torch CPU ops) of the reference's decode layer, used ONLY as the timed
CPU baseline of bench.py (``cpu_baseline`` and ``--impl reference``).  Test infrastructure: the
product package never imports it.

It follows the reference's off-CUDA code path for a token step: ``attn_step_batched`` /
``ffn_step_batched`` (rwkv7_hf/native.py:180-280) with every projection an int4 group-128 linear
evaluated the way the reference does on CPU: unpack nibbles, materialise the dense weight, ``F.linear``
(rwkv7_hf/sm70_quant.py:598-610).  Activations are fp32 (the reference's CPU configuration).
Checked against the NumPy oracle in tests/test_cpu_port.py.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

EXP_HALF = 0.606531


def quantize_w4_groupwise(weight, group_size=128):
    w = weight.float()
    O, K = w.shape
    g = w.reshape(O, K // group_size, group_size)
    s = (g.abs().amax(dim=2) / 7).clamp_min(1e-6)
    q = (g / s[:, :, None]).round().clamp(-7, 7).to(torch.int16) + 8
    q = q.reshape(O, K)
    return ((q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)).contiguous(), s.contiguous()


def w4_groupwise_linear(x, packed, scales, group_size=128):
    O, K = packed.shape[0], packed.shape[1] * 2
    lo = (packed & 15).to(x.dtype) - 8
    hi = (packed >> 4).to(x.dtype) - 8
    w = torch.empty(O, K, dtype=x.dtype)
    w[:, 0::2] = lo
    w[:, 1::2] = hi
    return F.linear(x, w * scales.to(x.dtype).repeat_interleave(group_size, dim=1))


def make_layer(D, H, N, Fdim, ranks, layer_id, seed, group_size=128):
    """Random 7.2B-style layer: quantised r/k/v/o/key/value, dense LoRA and vectors."""
    g = torch.Generator().manual_seed(seed)
    A = H * N
    rn = lambda *s, std=0.02: torch.randn(*s, generator=g) * std
    p = {}
    for name, (o, i) in dict(Rw=(A, D), Kw=(A, D), Vw=(A, D), Ow=(D, A), fK=(Fdim, D), fV=(D, Fdim)).items():
        p[name] = quantize_w4_groupwise(rn(o, i), group_size)
    rw, ra, rv, rg = ranks
    p.update(w1=rn(rw, D), w2=rn(A, rw), w0=-5 + 4 * torch.rand(A, generator=g),
             a1=rn(ra, D), a2=rn(A, ra), a0=rn(A, std=0.5), g1=rn(rg, D), g2=rn(A, rg),
             v1=rn(rv, D), v2=rn(A, rv), v0=rn(A, std=0.5))
    for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g", "fx_k"):
        p[n] = torch.rand(D, generator=g)
    p.update(k_k=0.85 + rn(A, std=0.1), k_a=1 + rn(A, std=0.1), r_k=rn(H, N, std=0.1),
             gn_w=1 + rn(A, std=0.1), gn_b=rn(A, std=0.1),
             attn_w=1 + rn(D, std=0.1), attn_b=rn(D, std=0.1), ffn_w=1 + rn(D, std=0.1), ffn_b=rn(D, std=0.1))
    p["layer_id"] = layer_id
    return p


def layer_step(p, x, xpa, xpf, v_first, state, H, N):
    """One layer, one token, batch B.  Returns (x, xpa, xpf, v_first, state)."""
    B, D = x.shape
    A = H * N
    lin = lambda t, name: w4_groupwise_linear(t, *p[name])
    h = F.layer_norm(x, (D,), p["attn_w"], p["attn_b"], 1e-5)
    xx = xpa - h
    xr, xw, xk, xv, xa, xg = (h + xx * p[n] for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"))
    r, k, v = lin(xr, "Rw"), lin(xk, "Kw"), lin(xv, "Vw")
    w = F.linear(torch.tanh(F.linear(xw, p["w1"])), p["w2"], p["w0"])
    a = torch.sigmoid(F.linear(F.linear(xa, p["a1"]), p["a2"], p["a0"]))
    g = F.linear(torch.sigmoid(F.linear(xg, p["g1"])), p["g2"])
    kk = F.normalize((k * p["k_k"]).view(B, H, N), dim=-1, p=2).view(B, A)
    k = k * (1 + (a - 1) * p["k_a"])
    if p["layer_id"] == 0:
        v_first = v
    else:
        v = v + (v_first - v) * torch.sigmoid(F.linear(F.linear(xv, p["v1"]), p["v2"], p["v0"]))
    w = torch.exp(-EXP_HALF * torch.sigmoid(w))
    vk = v.view(B, H, N, 1) @ k.view(B, H, 1, N)
    ab = (-kk).view(B, H, N, 1) @ (kk * a).view(B, H, 1, N)
    state = state * w.view(B, H, 1, N) + state @ ab + vk
    out = (state @ r.view(B, H, N, 1)).view(B, A)
    out = F.group_norm(out, H, p["gn_w"], p["gn_b"], N * 1e-5)
    sk = (r.view(B, H, N) * k.view(B, H, N) * p["r_k"]).sum(-1, keepdim=True)
    out = out + (sk * v.view(B, H, N)).view(B, A)
    x = x + lin(out * g, "Ow")
    h2 = F.layer_norm(x, (D,), p["ffn_w"], p["ffn_b"], 1e-5)
    kx = h2 + (xpf - h2) * p["fx_k"]
    x = x + lin(torch.relu(lin(kx, "fK")) ** 2, "fV")
    return x, h, h2, v_first, state


def head_step(x, norm_w, norm_b, head_w):
    return F.linear(F.layer_norm(x, (x.shape[1],), norm_w, norm_b, 1e-5), head_w)
