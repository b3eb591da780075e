"""The timed CPU baseline (`oracle/dense_torch.py`, the leg `bench.py` reports as `cpu_baseline` and runs for
`--impl reference`) against the reference's own dense solver: `fix_f` / `fix_g` of `dense_reference.npz` were
produced by the reference's `sinkhorn_geomloss_potentials_ref` (testing/reference_sinkhorn.py:119-192) with a
fixed eps of 0.3, 20 iterations and no final extrapolation - exactly init + 20 averaged Jacobi steps."""
import numpy as np
import torch

from oracle import dense_torch
from tests.conftest import load_golden, rel_err


def _inputs():
    z = load_golden("dense_reference")
    return z, [torch.from_numpy(z[k]) for k in ("x", "y", "a", "b")]


def test_cpu_baseline_port_matches_reference_dense_solver():
    z, (x, y, a, b) = _inputs()
    f, g, seconds, entries = dense_torch.symmetric_steps(x, y, a, b, 0.3, 20)
    assert rel_err(f.numpy(), z["fix_f"]) < 3e-5
    assert rel_err(g.numpy(), z["fix_g"]) < 3e-5
    assert entries == 2 * x.shape[0] * y.shape[0] * 21 and seconds > 0.0


def test_cpu_baseline_port_row_chunking_does_not_change_the_result():
    _, (x, y, a, b) = _inputs()
    f0, g0, _, _ = dense_torch.symmetric_steps(x, y, a, b, 0.3, 5, chunk=4096)
    f1, g1, _, _ = dense_torch.symmetric_steps(x, y, a, b, 0.3, 5, chunk=37)
    assert np.allclose(f0.numpy(), f1.numpy(), rtol=0, atol=2e-6)
    assert np.allclose(g0.numpy(), g1.numpy(), rtol=0, atol=2e-6)


def test_cpu_baseline_port_cost_scale_is_input_scaling():
    _, (x, y, a, b) = _inputs()
    f0, g0, _, _ = dense_torch.symmetric_steps(x, y, a, b, 0.3, 5, cost_scale=0.5)
    s = 0.5 ** 0.5
    f1, g1, _, _ = dense_torch.symmetric_steps(s * x, s * y, a, b, 0.3, 5)
    assert np.allclose(f0.numpy(), f1.numpy(), atol=5e-6) and np.allclose(g0.numpy(), g1.numpy(), atol=5e-6)
