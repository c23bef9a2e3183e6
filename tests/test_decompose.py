"""Parity study of the randomised decomposition (`svd="randomized"`) against the reference's full-SVD recipe
(bitstack/modules/BitStackLinear.py:49-75, which `svd="full"` follows line by line).

The randomised variant is NOT bit-compatible with the full SVD, so it is judged by what the decomposition is for:
the residual that is left after every block, and the output of the layer built from it.
"""
import numpy as np
import pytest
import torch

from bitstack_b200.linear import BitStackLinear, truncated_svd
from bitstack_b200.pack import unpack_sign


def _dense_from_blocks(mod, nb, m, n):
    """float64 weight of the first nb blocks, from the module's packed buffers (on their device)."""
    w = torch.zeros(m, n, dtype=torch.float64, device=mod.u_0.device)
    for j in range(nb):
        sign = unpack_sign(getattr(mod, f"qweight_{j}"), (m, n)).double()
        w += sign * (getattr(mod, f"u_{j}").double() @ getattr(mod, f"vt_{j}").double())
    return w


def _residuals(weight, mod, nb):
    m, n = weight.shape
    return [float((weight.double() - _dense_from_blocks(mod, j + 1, m, n)).norm()) for j in range(nb)]


def _residual_recursion(weight, nb, k, svd):
    """The decomposition recipe without the packed storage (pure torch, runs on the CPU): residual norms per block."""
    w = weight.clone().float()
    out = []
    for _ in range(nb):
        sign = w.sign()
        sign[sign == 0] = 1
        u, s, vt = svd(w.abs())
        w = w - sign * ((u[:, :k] * s[:k]) @ vt[:k])
        out.append(float(w.norm()))
    return out


def test_truncated_svd_leading_triplets_cpu():
    torch.manual_seed(0)
    a = (torch.randn(384, 640) * 0.02).abs()
    u, s, vt = torch.linalg.svd(a, full_matrices=False)
    g = torch.Generator().manual_seed(1)
    u2, s2, vt2 = truncated_svd(a, 16, oversample=16, power_iters=4, generator=g)
    assert u2.shape == (384, 16) and s2.shape == (16,) and vt2.shape == (16, 640)
    # the dominant (Perron) triplet is exact to fp32 accuracy, the flat tail of a random matrix converges slowly
    assert abs(float(s2[0] - s[0])) <= 1e-5 * float(s[0])
    assert float(((s2 - s[:16]).abs() / s[:16]).max()) <= 0.06
    # what matters: the rank-16 approximation is as good as the optimal one to a fraction of a percent
    best = float((a - (u[:, :16] * s[:16]) @ vt[:16]).norm())
    got = float((a - (u2 * s2) @ vt2).norm())
    assert best <= got <= 1.005 * best
    # orthonormal factors
    assert float((u2.t() @ u2 - torch.eye(16)).abs().max()) <= 1e-4
    assert float((vt2 @ vt2.t() - torch.eye(16)).abs().max()) <= 1e-4


def test_randomized_recursion_matches_full_svd_residuals_cpu():
    torch.manual_seed(3)
    w = torch.randn(192, 256) * 0.02
    g = torch.Generator().manual_seed(5)
    r_full = _residual_recursion(w, 4, 16, lambda a: torch.linalg.svd(a, full_matrices=False))
    r_rnd = _residual_recursion(w, 4, 16, lambda a: truncated_svd(a, 16, generator=g))
    for a, b in zip(r_full, r_rnd):
        assert b <= 1.01 * a, (r_full, r_rnd)
    assert r_rnd[-1] < r_rnd[0] < float(w.norm())


@pytest.mark.gpu
def test_randomized_decomposition_on_the_device_forward_and_residuals():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    torch.manual_seed(11)
    m, n, nb = 2048, 2048, 6
    lin = torch.nn.Linear(n, m, bias=False).to(dev)
    lin.weight.data = (torch.randn(m, n, device=dev) * 0.02)
    full = BitStackLinear.from_linear(lin, w_bit=nb, k=16, bias=False, fused_level=6)
    rnd = BitStackLinear.from_linear(lin, w_bit=nb, k=16, bias=False, fused_level=6, svd="randomized", seed=2)
    r_full, r_rnd = _residuals(lin.weight.data, full, nb), _residuals(lin.weight.data, rnd, nb)
    for a, b in zip(r_full, r_rnd):
        assert b <= 1.01 * a, (r_full, r_rnd)
    # the first block's signs are those of W itself in both; the randomised variant is deterministic for a seed
    assert torch.equal(full.qweight_0, rnd.qweight_0)
    again = BitStackLinear.from_linear(lin, w_bit=nb, k=16, bias=False, fused_level=6, svd="randomized", seed=2)
    for j in range(nb):
        assert torch.equal(getattr(rnd, f"u_{j}"), getattr(again, f"u_{j}"))
        assert torch.equal(getattr(rnd, f"qweight_{j}"), getattr(again, f"qweight_{j}"))
    with pytest.raises(ValueError):
        BitStackLinear.from_linear(lin, w_bit=1, k=16, bias=False, svd="lanczos")
    # the layer built from the randomised factors is as close to the dense layer as the one from the full SVD
    x = torch.randn(4, n, device=dev).half()
    y_dense = (x.float() @ lin.weight.data.t()).cpu().numpy()
    full.stack_blocks()
    rnd.stack_blocks()
    e_full = np.linalg.norm(full(x).float().cpu().numpy() - y_dense) / np.linalg.norm(y_dense)
    e_rnd = np.linalg.norm(rnd(x).float().cpu().numpy() - y_dense) / np.linalg.norm(y_dense)
    assert e_rnd <= 1.02 * e_full + 1e-4, (e_full, e_rnd)
