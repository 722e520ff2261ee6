"""Helpers for the GPU parity tests (imported by the test modules, not collected)."""
import os

import numpy as np
import torch

DEV = "cuda"


def golden(name):
    here = os.path.dirname(os.path.abspath(__file__))
    return dict(np.load(os.path.join(here, "golden", name)))


def cu(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def npf(t):
    return t.detach().float().cpu().numpy()


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def wkv_inputs(B, T, H, N, seed, dtype=np.float16):
    """Config-2 style inputs: r,k,v ~ N(0,1); kk = normalised k; a = sigmoid(g); w = exp(-0.606531*sigmoid(z))."""
    rng = np.random.default_rng(seed)
    r, k, v = (rng.standard_normal((B, T, H, N)).astype(dtype) for _ in range(3))
    kf = k.astype(np.float32)
    kk = (kf / np.maximum(np.linalg.norm(kf, axis=-1, keepdims=True), 1e-12)).astype(dtype)
    a = (1 / (1 + np.exp(-rng.standard_normal((B, T, H, N))))).astype(dtype)
    w = np.exp(-0.606531 / (1 + np.exp(-rng.standard_normal((B, T, H, N))))).astype(np.float32)
    return r, w, k, v, kk, a
