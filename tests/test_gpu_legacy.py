"""OTT-convention legacy surface on the GPU (signed log-sum-exp, half-steps, deprecated plan applications and
solver facades) against fixtures made by the reference and against the CPU oracle."""
import warnings

import numpy as np
import pytest
import torch

from conftest import load_golden
from gpu_util import MODES, TOL, dev, host, rel, set_mode
from oracle import dense_sinkhorn as O

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _signed_close(out, sgn, x, y, f, g, eps, axis, vec, tol):
    """out = level + eps*log|r| with r the softmax-weighted mean of vec: an error dr in r moves out by
    eps*dr/|r|, so the budget per entry scales with 1/|r|."""
    want, want_sgn = O.signed_lse_ott(x, y, f, g, eps, axis, vec=vec)
    level, _ = O.signed_lse_ott(x, y, f, g, eps, axis)
    r = np.exp((want - level) / eps)
    budget = eps * tol * np.abs(vec).max() / np.maximum(r, 1e-30) + tol * (1.0 + np.abs(want))
    assert np.all(np.abs(out - want) <= budget), float((np.abs(out - want) / budget).max())
    firm = r > 10 * tol * np.abs(vec).max()  # the sign is only determined where r is clear of the noise
    assert np.array_equal(sgn[firm], want_sgn[firm])


@pytest.mark.parametrize("mode", MODES)
def test_signed_lse_and_half_steps_vs_reference(monkeypatch, mode):
    from flash_sinkhorn_b200.kernels.sinkhorn_triton_ott_sqeuclid import (
        apply_lse_kernel_sqeuclid, apply_transport_from_potentials_sqeuclid, update_potential)
    set_mode(monkeypatch, mode)
    tol = TOL[mode]
    z = load_golden("legacy_ott_small")
    eps = float(z["eps"])
    x, y, f, g, vm, vn, la, lb = (dev(z[k]) for k in ("x", "y", "f", "g", "vec_m", "vec_n", "loga", "logb"))
    z64 = {k: z[k].astype(np.float64) for k in ("x", "y", "f", "g", "vec_m", "vec_n")}
    for axis, vec, vkey in ((1, vm, "vec_m"), (0, vn, "vec_n")):
        out, sgn = apply_lse_kernel_sqeuclid(x, y, f, g, eps, axis)
        assert rel(host(out), z[f"lse_axis{axis}"]) < tol and bool((sgn == 1).all())
        out, sgn = apply_lse_kernel_sqeuclid(x, y, f, g, eps, axis, vec=vec)
        _signed_close(host(out), host(sgn), z64["x"], z64["y"], z64["f"], z64["g"], eps, axis, z64[vkey], tol)
        if mode != "tf32":
            assert np.array_equal(host(sgn), z[f"vlse_sgn_axis{axis}"])
            assert np.abs(host(out) - z[f"vlse_axis{axis}"]).max() < 2e-3
    out, sgn = apply_lse_kernel_sqeuclid(x, y, f, g, eps, 1, vec=torch.zeros_like(vm))
    assert bool(torch.isneginf(out).all()) and bool((sgn == 0).all())
    # given squared norms are used as they are
    out2, _ = apply_lse_kernel_sqeuclid(x, y, f, g, eps, 1, x2=(x * x).sum(1), y2=(y * y).sum(1))
    assert rel(host(out2), z["lse_axis1"]) < tol

    assert rel(host(update_potential(x, y, f, g, lb, eps, axis=0)), z["update_g"]) < tol
    assert rel(host(update_potential(x, y, f, g, la, eps, axis=1)), z["update_f"]) < tol
    fo, go = dev(z["ott_f_dense"]), dev(z["ott_g_dense"])
    assert rel(host(apply_transport_from_potentials_sqeuclid(x, y, fo, go, vm, eps, 1)), z["transport_axis1"]) < tol
    assert rel(host(apply_transport_from_potentials_sqeuclid(x, y, fo, go, vn, eps, 0)), z["transport_axis0"]) < tol


@pytest.mark.parametrize("mode", MODES)
def test_signed_lse_medium_vs_oracle(monkeypatch, mode):
    """Several row blocks and column tiles, fp16 inputs (converted to fp32 as in the reference), masked
    (-inf) potentials on the summed side."""
    from flash_sinkhorn_b200.kernels.sinkhorn_triton_ott_sqeuclid import apply_lse_kernel_sqeuclid
    set_mode(monkeypatch, mode)
    tol = TOL[mode]
    gen = torch.Generator().manual_seed(5)
    n, m, d, eps = 700, 900, 32, 0.8
    x = (0.5 * torch.randn(n, d, generator=gen)).half()
    y = (0.5 * torch.randn(m, d, generator=gen)).half()
    f, g = torch.randn(n, generator=gen), torch.randn(m, generator=gen)
    g[::7] = float("-inf")
    vec = torch.randn(n, generator=gen)
    x64, y64 = x.double().numpy(), y.double().numpy()
    f64, g64 = f.double().numpy(), g.double().numpy()
    out, sgn = apply_lse_kernel_sqeuclid(x.cuda(), y.cuda(), f.cuda(), g.cuda(), eps, 1)
    want, _ = O.signed_lse_ott(x64, y64, f64, g64, eps, 1)
    assert rel(host(out), want) < tol and bool((sgn == 1).all())
    out, sgn = apply_lse_kernel_sqeuclid(x.cuda(), y.cuda(), f.cuda(), g.cuda(), eps, 0, vec=vec.cuda())
    keep = np.isfinite(g64)  # masked columns: the reference itself returns NaN there (inf - inf), nothing to pin
    want, want_sgn = O.signed_lse_ott(x64, y64[keep], f64, g64[keep], eps, 0, vec=vec.double().numpy())
    level, _ = O.signed_lse_ott(x64, y64[keep], f64, g64[keep], eps, 0)
    r = np.exp((want - level) / eps)
    got, got_sgn = host(out)[keep], host(sgn)[keep]
    budget = eps * tol * np.abs(vec.numpy()).max() / np.maximum(r, 1e-30) + tol * (1.0 + np.abs(want))
    assert np.all(np.abs(got - want) <= budget)
    firm = r > 10 * tol * np.abs(vec.numpy()).max()
    assert np.array_equal(got_sgn[firm], want_sgn[firm])


@pytest.mark.parametrize("mode", MODES)
def test_deprecated_ott_wrappers_vs_reference(monkeypatch, mode):
    from flash_sinkhorn_b200.kernels import sinkhorn_triton_apply_sqeuclid as shim
    from flash_sinkhorn_b200.kernels.apply_ott import apply_plan_mat_sqeuclid, apply_plan_vec_sqeuclid
    from flash_sinkhorn_b200.kernels.sinkhorn_triton_geomloss_sqeuclid import (
        sinkhorn_geomloss_online_potentials_sqeuclid)
    from flash_sinkhorn_b200.kernels.sinkhorn_triton_ott_sqeuclid import sinkhorn_potentials_sqeuclid
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
    set_mode(monkeypatch, mode)
    tol = TOL[mode]
    z = load_golden("legacy_ott_small")
    eps, cs = float(z["eps"]), float(z["cs"])
    x, y, vm, vn, la, lb, fh, gh, mm, mn, sc = (dev(z[k]) for k in (
        "x", "y", "vec_m", "vec_n", "loga", "logb", "cs_f", "cs_g", "mat_m", "mat_n", "scale"))
    assert shim.apply_plan_vec_sqeuclid is apply_plan_vec_sqeuclid
    with pytest.warns(DeprecationWarning):
        got = apply_plan_vec_sqeuclid(x, y, fh, gh, vm, eps=eps, axis=1, cost_scale=cs, log_a=la, log_b=lb)
    assert rel(host(got), z["dep_vec_axis1"]) < tol
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", DeprecationWarning)
        got = apply_plan_vec_sqeuclid(x, y, fh, gh, vn, eps=eps, axis=0, cost_scale=cs)
        assert rel(host(got), z["dep_vec_axis0"]) < tol
        got = apply_plan_mat_sqeuclid(x, y, fh, gh, mm, eps=eps, axis=1, cost_scale=cs, scale=sc, log_a=la, log_b=lb)
        assert rel(host(got), z["dep_mat_axis1"]) < tol
        got = apply_plan_mat_sqeuclid(x, y, fh, gh, mn, eps=eps, axis=0, cost_scale=cs)
        assert rel(host(got), z["dep_mat_axis0"]) < tol
        with pytest.raises(ValueError):
            apply_plan_mat_sqeuclid(x, y, fh, gh, mn, eps=eps, axis=0, scale=sc)
        with pytest.raises(ValueError):
            apply_plan_vec_sqeuclid(x, y, fh, gh, vn, eps=eps, axis=1)
    with pytest.warns(DeprecationWarning):
        ff, gf = sinkhorn_potentials_sqeuclid(x, y, la, lb, eps, 6)
    assert rel(host(ff), z["ott_f_facade"]) < tol and rel(host(gf), z["ott_g_facade"]) < tol
    a, b = torch.exp(la), torch.exp(lb)
    with pytest.warns(DeprecationWarning):
        old = sinkhorn_geomloss_online_potentials_sqeuclid(x, y, a, b, blur=0.5, scaling=0.7, block_m=64)
    new = sinkhorn_flashstyle_symmetric(x, y, a, b, blur=0.5, scaling=0.7)
    assert torch.equal(old[0], new[0]) and torch.equal(old[1], new[1])

