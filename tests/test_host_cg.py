"""Host-driven Krylov solvers of flash_sinkhorn_b200.cg on CPU tensors (they take any matvec callable):
the trust-region CG against fixtures made by the reference's steihaug_cg, plain CG against a dense solve."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from flash_sinkhorn_b200.cg import SteihaugCGInfo, conjugate_gradient, steihaug_cg


@pytest.mark.parametrize("name", ["interior", "boundary", "negcurv", "maxiter"])
def test_steihaug_vs_reference(name):
    z = load_golden("steihaug_small")
    H, g = torch.from_numpy(z[name + "_H"]), torch.from_numpy(z[name + "_g"])
    delta, max_iter, rtol = z[name + "_args"]
    p, info = steihaug_cg(lambda v: H @ v, g, float(delta), max_iter=int(max_iter), rtol=float(rtol), atol=1e-12)
    assert isinstance(info, SteihaugCGInfo)
    conv, iters, resid, hit, neg, red = z[name + "_info"]
    assert info.termination_reason == str(z[name + "_reason"])
    assert (info.converged, info.iters, info.hit_boundary, info.negative_curvature_detected) == (
        bool(conv), int(iters), bool(hit), bool(neg))
    assert np.abs(p.numpy() - z[name + "_p"]).max() < 1e-10
    assert abs(info.residual - resid) < 1e-10 and abs(info.predicted_reduction - red) < 1e-9
    if info.hit_boundary:
        assert abs(float(p.norm()) - float(delta)) < 1e-8


def test_steihaug_zero_gradient_and_model_decrease():
    p, info = steihaug_cg(lambda v: v, torch.zeros(7), 1.0)
    assert info.converged and info.iters == 0 and float(p.abs().max()) == 0.0
    gen = torch.Generator().manual_seed(3)
    B = torch.randn(20, 20, generator=gen, dtype=torch.float64)
    H = 0.5 * (B + B.T)  # indefinite
    g = torch.randn(20, generator=gen, dtype=torch.float64)
    for delta in (0.1, 1.0, 10.0):
        p, info = steihaug_cg(lambda v: H @ v, g, delta)
        assert float(p.norm()) <= delta * (1 + 1e-9)
        model = float(g @ p + 0.5 * p @ (H @ p))
        assert model < 0 and abs(-model - info.predicted_reduction) < 1e-9


def test_conjugate_gradient_dense_spd():
    gen = torch.Generator().manual_seed(4)
    B = torch.randn(40, 40, generator=gen, dtype=torch.float64)
    A = B @ B.T / 40 + 0.3 * torch.eye(40, dtype=torch.float64)
    b = torch.randn(40, generator=gen, dtype=torch.float64)
    sol, info = conjugate_gradient(lambda v: A @ v, b, rtol=1e-10, atol=0.0)
    assert info.cg_converged and float((A @ sol - b).norm()) <= 1e-10 * float(b.norm()) * 1.01
    sol2, info2 = conjugate_gradient(lambda v: A @ v, b, max_iter=3)
    assert not info2.cg_converged and info2.cg_iters == 3
    dinv = 1.0 / torch.diagonal(A)
    sol3, info3 = conjugate_gradient(lambda v: A @ v, b, rtol=1e-10, atol=0.0, preconditioner=lambda r: dinv * r,
                                     x0=sol2, stabilise_every=5)
    assert info3.cg_converged and float((sol3 - sol).norm()) < 1e-8
