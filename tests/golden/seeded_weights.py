"""Seeded weights for model-level fixtures that are too large to store.

``seeded_state_dict`` fills every entry of an RWKV-7 ``state_dict`` (reference naming:
``model.layers.N.attn.r_proj.weight`` ...) from a generator keyed by the entry's name, so the fixture generator
(which loads the result into the reference model) and the parity tests (which load it into this package's model)
build bit-identical weights without the reference, and the fixture stores only a checksum.  The distributions
follow what a trained RWKV-7 looks like closely enough that every term of the recurrence carries weight: the
reference constructs the token-shift and key-scale parameters as zeros (rwkv7_hf/model_layers.py:54-58,109), which
would switch the delta-rule term off.
"""
from __future__ import annotations

import zlib

import numpy as np
import torch


def _gen(name: str, seed: int) -> torch.Generator:
    return torch.Generator().manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 31 - 1))


def seeded_tensor(name: str, shape, seed: int) -> torch.Tensor:
    g = _gen(name, seed)
    shape = tuple(int(s) for s in shape)
    rn = lambda: torch.randn(shape, generator=g)
    ru = lambda: torch.rand(shape, generator=g)
    leaf = name.split(".")
    if leaf[-1] in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
        return ru()
    if leaf[-1] == "k_k":
        return 0.85 + 0.1 * rn()
    if leaf[-1] == "k_a":
        return 1.0 + 0.1 * rn()
    if leaf[-1] == "r_k":
        return 0.1 * rn()
    if "norm" in leaf[-2]:  # LayerNorm / GroupNorm affine parameters
        return 1.0 + 0.1 * rn() if leaf[-1] == "weight" else 0.1 * rn()
    if ".lora." in name:
        if leaf[-1] == "bias":
            return -5.0 + 4.0 * ru() if "w_lora" in name else 0.5 * rn()
        return 0.05 * rn()
    if leaf[-2] == "embeddings":
        return rn()
    if leaf[-1] == "weight" and len(shape) == 2:
        return 0.02 * rn()
    if leaf[-1] == "bias":
        return torch.zeros(shape)
    raise KeyError(f"no recipe for {name} {shape}")


def seeded_state_dict(shapes: dict, seed: int, dtype=torch.float32) -> dict:
    """``shapes``: name -> shape (e.g. ``{k: v.shape for k, v in model.state_dict().items()}``)."""
    return {name: seeded_tensor(name, shape, seed).to(dtype) for name, shape in sorted(shapes.items())}


def checksum(sd: dict) -> np.ndarray:
    """[sum, sum of squares, number of values] over all entries in name order, in float64."""
    s = q = n = 0.0
    for name in sorted(sd):
        t = sd[name].detach().double()
        s += float(t.sum())
        q += float((t * t).sum())
        n += t.numel()
    return np.array([s, q, n], np.float64)
