"""The torch-CPU port used for the timed CPU baseline computes the same layer step as the pinned oracle."""
import numpy as np
import torch

from oracle import cpu_port_torch as P
from oracle import rwkv7_oracle as O


def test_cpu_port_layer_matches_oracle():
    D, H, N, Fd, B = 256, 2, 64, 512, 3
    torch.manual_seed(0)
    for layer_id in (0, 1):
        p = P.make_layer(D, H, N, Fd, (16, 16, 8, 32), layer_id, seed=layer_id + 5)
        x, xpa, xpf = torch.randn(B, D), torch.randn(B, D), torch.randn(B, D)
        vf, st = torch.randn(B, H * N), 0.3 * torch.randn(B, H, N, N)
        x1, xpa1, xpf1, vf1, st1 = P.layer_step(p, x, xpa, xpf, vf, st, H, N)
        n = lambda t: t.numpy()
        q = {k: (dict(kind="w4g", packed=n(v[0]), scales=n(v[1])) if isinstance(v, tuple) else (n(v) if torch.is_tensor(v) else v))
             for k, v in p.items()}
        xo, xpao, xpfo, vfo, sto = O.block_step(q, layer_id, n(x), n(xpa), n(xpf), n(vf), n(st), H, N)
        np.testing.assert_allclose(n(x1), xo, rtol=2e-4, atol=2e-4)
        np.testing.assert_allclose(n(st1), sto, rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(n(xpa1), xpao, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(n(xpf1), xpfo, rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(n(vf1), vfo, rtol=2e-4, atol=2e-5)
