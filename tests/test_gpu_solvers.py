"""Solver / SamplesLoss / HVP parity on the GPU against fixtures made by the reference and the CPU oracle."""
import os

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


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name,cs,rx,ry", [("bal_sched", 1.0, None, None), ("half_semi", 0.5, 1.0, None),
                                           ("unbal", 1.0, 1.0, 4.0)])
def test_symmetric_solver_vs_reference(monkeypatch, mode, name, cs, rx, ry):
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
    set_mode(monkeypatch, mode)
    z = load_golden("solvers_small")
    x, y, a, b = (dev(z[k]) for k in ("x", "y", "a", "b"))
    f, g, fp, gp, k = sinkhorn_flashstyle_symmetric(x, y, a, b, blur=0.3, scaling=0.6, cost_scale=cs, rho_x=rx,
                                                    rho_y=ry, return_prelast=True, return_n_iters=True)
    tag = f"sym_{name}_fused"
    assert k == int(z[tag + "_iters"])
    tol = TOL[mode]
    for got, key in ((f, "_f"), (g, "_g"), (fp, "_fpre"), (gp, "_gpre")):
        assert rel(host(got), z[tag + key]) < tol, key


@pytest.mark.parametrize("mode", MODES)
def test_symmetric_early_stop_and_warm_start(monkeypatch, mode):
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
    set_mode(monkeypatch, mode)
    z = load_golden("solvers_small")
    x, y, a, b = (dev(z[k]) for k in ("x", "y", "a", "b_normalised"))
    f, g, k = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=5.0, n_iters=60,
                                            threshold=1e-3, check_every=4, return_n_iters=True)
    if mode != "tf32":  # the stopping iteration is a discrete function of rounding noise
        assert k == int(z["sym_early_iters"])
    assert k < 62
    assert rel(host(f), z["sym_early_f"]) < max(TOL[mode], 2e-3)
    f2, g2 = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=5.0, n_iters=3,
                                           f_init=dev(z["sym_early_f"]), g_init=dev(z["sym_early_g"]),
                                           last_extrapolation=False)
    assert rel(host(f2), z["sym_warm_f"]) < TOL[mode] and rel(host(g2), z["sym_warm_g"]) < TOL[mode]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("conv", [False, True])
@pytest.mark.parametrize("rho", [None, 2.0])
def test_alternating_solver_vs_reference(monkeypatch, mode, conv, rho):
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    set_mode(monkeypatch, mode)
    z = load_golden("solvers_small")
    x, y, a, b = (dev(z[k]) for k in ("x", "y", "a", "b"))
    f, g, k = sinkhorn_flashstyle_alternating(x, y, a, b, eps=0.4, n_iters=12, cost_scale=0.5, rho_x=rho, rho_y=rho,
                                              ott_convention=conv, return_n_iters=True)
    tag = f"alt_{'ott' if conv else 'geo'}_{'bal' if rho is None else 'unb'}"
    assert k == 12
    assert rel(host(f), z[tag + "_f"]) < TOL[mode] and rel(host(g), z[tag + "_g"]) < TOL[mode]


def test_alternating_early_stop_vs_reference(monkeypatch):
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    set_mode(monkeypatch, "fp32")
    z = load_golden("solvers_small")
    x, y, a, b = (dev(z[k]) for k in ("x", "y", "a", "b_normalised"))
    f, g, k = sinkhorn_flashstyle_alternating(x, y, a, b, eps=5.0, n_iters=80, threshold=1e-4, check_every=3,
                                              return_n_iters=True)
    assert k == int(z["alt_early_iters"])
    assert rel(host(f), z["alt_early_f"]) < 2e-4


def test_annealed_alternating_and_tile_mask_vs_oracle(monkeypatch):
    """Annealed alternating solve and block-sparse tile skipping (no reference implementation):
    checked against the dense masked oracle."""
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    set_mode(monkeypatch, "fp32")
    rng = np.random.default_rng(7)
    n, m, d = 300, 260, 3
    cx = rng.uniform(-1, 1, (4, d))
    lab_x, lab_y = np.sort(rng.integers(0, 4, n)), np.sort(rng.integers(0, 4, m))
    x = (cx[lab_x] + 0.05 * rng.standard_normal((n, d))).astype(np.float32)
    y = (cx[lab_y] + 0.05 * rng.standard_normal((m, d))).astype(np.float32)
    a, b = np.full(n, 1.0 / n, np.float32), np.full(m, 1.0 / m, np.float32)
    sched = O.epsilon_schedule(O.max_diameter(x, y), 0.05, 0.5)
    ref = O.solve_alternating(x.astype(np.float64), y.astype(np.float64), a.astype(np.float64), b.astype(np.float64),
                              sched, 4)
    f, g = sinkhorn_flashstyle_alternating(dev(x), dev(y), dev(a), dev(b), eps_list=sched, iters_per_eps=4)
    assert rel(host(f), ref["f"]) < 5e-4 and rel(host(g), ref["g"]) < 5e-4
    mask = np.ones(((n + 127) // 128, (m + 127) // 128), bool)
    mask[0, 2] = mask[2, 0] = mask[1, 2] = False
    ref = O.solve_alternating(x.astype(np.float64), y.astype(np.float64), a.astype(np.float64), b.astype(np.float64),
                              sched[:6], 3, tile_mask=mask)
    f, g = sinkhorn_flashstyle_alternating(dev(x), dev(y), dev(a), dev(b), eps_list=sched[:6], iters_per_eps=3,
                                           tile_mask=torch.as_tensor(mask))
    assert rel(host(f), ref["f"]) < 5e-4 and rel(host(g), ref["g"]) < 5e-4


LOSS_CFG = {
    "bal_debias_half": dict(blur=0.5, scaling=0.7, debias=True, half_cost=True),
    "bal_fixed": dict(blur=0.6, use_epsilon_scaling=False, eps=0.36, n_iters=25),
    "semi": dict(blur=0.5, scaling=0.7, reach_x=1.5),
    "unbal": dict(blur=0.5, scaling=0.7, reach=1.2, normalize=False),
    "alt": dict(backend="alternating", use_epsilon_scaling=False, eps=0.3, n_iters=15, blur=0.5),
}


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", sorted(LOSS_CFG))
def test_samples_loss_forward_backward_vs_reference(monkeypatch, mode, name):
    from flash_sinkhorn_b200 import SamplesLoss
    set_mode(monkeypatch, mode)
    z = load_golden("samples_loss_small")
    x, y, a, b = (dev(z[k]) for k in ("x", "y", "a", "b"))
    xs, ys, a_s = x.clone().requires_grad_(True), y.clone().requires_grad_(True), a.clone().requires_grad_(True)
    val = SamplesLoss("sinkhorn", **LOSS_CFG[name])(a_s, xs, b, ys)
    gx, gy, ga = torch.autograd.grad(val, (xs, ys, a_s))
    want = float(z[name + "_loss"])
    # Loss: rel 1e-4 in TF32 mode, 2e-5 in the fp32 modes. Gradients: 3e-4 (max-norm relative) in the
    # fp32 modes. In TF32 mode the fixture (made by the reference with fp32 products) is not the yardstick
    # for point gradients: rounding x, y to 11 significant bits perturbs every logit by ~|x||y| 2^-11 2cs/eps
    # (1e-2 here), which moves soft-min weights by the same relative amount in ANY TF32 implementation.
    ltol, gtol = (1e-4, 3e-2) if mode == "tf32" else (2e-5, 3e-4)
    assert abs(val.item() - want) <= ltol * max(1.0, abs(want))
    assert rel(host(gx), z[name + "_gx"]) < gtol
    assert rel(host(gy), z[name + "_gy"]) < gtol
    assert rel(host(ga), z[name + "_ga"]) < (2e-3 if mode == "tf32" else gtol)
    f, g = SamplesLoss("sinkhorn", potentials=True, **LOSS_CFG[name])(a, x, b, y)
    assert rel(host(f), z[name + "_f"]) < TOL[mode] and rel(host(g), z[name + "_g"]) < TOL[mode]


def test_samples_loss_call_forms_and_batches():
    from flash_sinkhorn_b200 import SamplesLoss
    z = load_golden("samples_loss_small")
    x, y = dev(z["x"]), dev(z["y"])
    loss = SamplesLoss("sinkhorn", blur=0.5, scaling=0.7, allow_tf32=False)
    v = loss(x, y)
    assert abs(v.item() - float(z["xy_loss"])) < 2e-5 * abs(float(z["xy_loss"]))
    n, m = x.shape[0], y.shape[0]
    a, b = torch.full((n, 1), 1.0 / n).cuda(), torch.full((m, 1), 1.0 / m).cuda()
    assert abs(loss(a, x, b, y).item() - v.item()) < 1e-6 * abs(v.item())  # (n,1) weights == uniform default
    xb, yb = torch.stack([x, x * 0.9]), torch.stack([y, y * 1.1])
    vb = loss(xb, yb)
    assert vb.shape == (2,) and abs(vb[0].item() - v.item()) < 1e-6 * abs(v.item())
    f, g = SamplesLoss("sinkhorn", blur=0.5, scaling=0.7, potentials=True)(a, x, b, y)
    assert f.shape == (n, 1) and g.shape == (m, 1)
    # debiased self-divergence vanishes (reference test_samples_loss_api.py:158-160)
    s = SamplesLoss("sinkhorn", blur=0.5, scaling=0.7, debias=True, allow_tf32=False)(x, x.clone())
    assert abs(s.item()) < 1e-4
    # half cost is half the full cost up to the eps change of scale (reference test_half_cost.py:21-33)
    full = SamplesLoss("sinkhorn", blur=0.05, allow_tf32=False)(x, y).item()
    half = SamplesLoss("sinkhorn", blur=0.05, half_cost=True, allow_tf32=False)(x, y).item()
    assert 1.95 < full / half < 2.05


@pytest.mark.parametrize("name,rx,ry,cs", [("bal", None, None, 1.0), ("semi_half", 2.0, None, 0.5)])
@pytest.mark.parametrize("mode", ["simt", "fp32"])
def test_hvp_vs_reference(monkeypatch, mode, name, rx, ry, cs):
    from flash_sinkhorn_b200.hvp import hvp_x_sqeuclid_from_potentials
    set_mode(monkeypatch, mode)
    z = load_golden("hvp_small")
    x, y, A = dev(z["x"]), dev(z["y"]), dev(z["A"])
    hv, info = hvp_x_sqeuclid_from_potentials(x, y, dev(z[name + "_f_ott"]), dev(z[name + "_g_ott"]), A,
                                              eps=float(z["eps"]), rho_x=rx, rho_y=ry, cost_scale=cs, max_cg_iter=400)
    assert info.cg_converged
    assert abs(info.cg_iters - int(z[name + "_cg"][1])) <= 3
    assert rel(host(hv), z[name + "_hvp"]) < 1e-3
    # host-driven CG path (warm start given) agrees with the device-resident loop
    hv2, info2 = hvp_x_sqeuclid_from_potentials(x, y, dev(z[name + "_f_ott"]), dev(z[name + "_g_ott"]), A,
                                                eps=float(z["eps"]), rho_x=rx, rho_y=ry, cost_scale=cs,
                                                max_cg_iter=400, cg_x0=torch.zeros(y.shape[0]).cuda())
    assert info2.cg_converged and rel(host(hv2), host(hv)) < 1e-3


def test_double_backward_equals_direct_hvp():
    """reference test_samples_loss_api.py:271-355."""
    from flash_sinkhorn_b200 import SamplesLoss
    from flash_sinkhorn_b200.hvp import hvp_x_sqeuclid
    z = load_golden("samples_loss_small")
    x, y, a, b, v = (dev(z[k]) for k in ("x", "y", "a", "b", "v"))
    xs = x.clone().requires_grad_(True)
    cfg = dict(blur=0.6, use_epsilon_scaling=False, eps=0.36, n_iters=25, allow_tf32=False, normalize=False)
    val = SamplesLoss("sinkhorn", **cfg)(a, xs, b, y)
    (gx,) = torch.autograd.grad(val, xs, create_graph=True)
    (hv,) = torch.autograd.grad((gx * v).sum(), xs)
    direct, info = hvp_x_sqeuclid(x, y, a, b, v, eps_list=[0.36] * 25, allow_tf32=False)
    assert info.cg_converged
    torch.testing.assert_close(hv, direct, rtol=1e-5, atol=1e-6)
    want = O.samples_loss(*(host(t) for t in (x, y, a, b)), [0.36] * 25)
    assert abs(val.item() - want["loss"]) < 2e-5 * abs(want["loss"])
    with pytest.raises(NotImplementedError):
        ys = y.clone().requires_grad_(True)
        val = SamplesLoss("sinkhorn", **cfg)(a, x, b, ys)
        (gy,) = torch.autograd.grad(val, ys, create_graph=True)
        torch.autograd.grad(gy.sum(), ys)


@pytest.mark.parametrize("allow_tf32", [False, True])
def test_config1_matches_reference_golden(allow_tf32):
    """Benchmark configuration 1: n=m=4096, d=64, eps=0.01, half cost, debias, 100 fixed iterations.
    Tolerances are the north-star ones: loss rel 1e-4, grad_x rel 1e-3 (of the gradient's max-norm)."""
    from flash_sinkhorn_b200 import SamplesLoss
    z = load_golden("config1")
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(4096, 64, generator=gen).cuda().requires_grad_(True)
    y = torch.randn(4096, 64, generator=gen).cuda()
    loss = SamplesLoss("sinkhorn", blur=0.1, use_epsilon_scaling=False, eps=0.01, n_iters=100, half_cost=True,
                       debias=True, allow_tf32=allow_tf32)
    val = loss(x, y)
    (gx,) = torch.autograd.grad(val, x)
    assert abs(val.item() - float(z["loss"])) <= 1e-4 * abs(float(z["loss"]))
    # Gradient as a whole (Frobenius norm): rel 1e-3 in both modes. Single entries: 1e-3 of the largest
    # entry in exact-fp32 (3xTF32) mode. In TF32 mode single entries at eps = 0.01 are ill-conditioned
    # for ANY TF32 implementation: rounding x, y to 11 bits moves each logit (= cost/eps) by ~0.3.
    assert abs(gx.norm().item() - float(z["grad_x_norm"])) <= 1e-3 * float(z["grad_x_norm"])
    assert rel(host(gx[:16]), z["grad_x_head"]) < (6e-2 if allow_tf32 else 1e-3)
    assert rel(host(gx.sum(dim=1)), z["grad_x_rowsum"]) < (1e-1 if allow_tf32 else 1e-3)


def test_marginals_at_scale_property():
    """Size-independent property at configuration-2 size (n=m=50,000, d=64): after a g-update of the
    alternating solver the column marginals of the plan equal b (reference test_flashstyle_parity.py:291-320)."""
    from flash_sinkhorn_b200.kernels._common import log_weights
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_vec_flashstyle
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    gen = torch.Generator().manual_seed(1)
    n = m = 50000
    x = torch.randn(n, 64, generator=gen).cuda()
    y = (0.5 + torch.randn(m, 64, generator=gen)).cuda()
    a, b = torch.full((n,), 1.0 / n).cuda(), torch.full((m,), 1.0 / m).cuda()
    eps = 0.5
    # Solve and plan application both run on the tensor-core engine over the same staged operands, so the
    # scores are bit-identical and the identity holds to the TF32 rounding of the weights (2^-12, averaged).
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle
    f, g = sinkhorn_flashstyle_alternating(x, y, a, b, eps=eps, n_iters=3, allow_tf32=True)
    fh, gh = f - (x**2).sum(1), g - (y**2).sum(1)
    col = apply_plan_mat_flashstyle(x, y, fh, gh, log_weights(a), log_weights(b), torch.ones(n, 64).cuda(), eps=eps,
                                    axis=0, allow_tf32=True)[:, 0].contiguous()
    assert torch.isfinite(col).all()
    assert (col / b - 1).abs().max().item() < 5e-3
    assert abs(col.sum().item() - 1.0) < 1e-3


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("threshold", [None, 1e-3])
def test_self_transport_shortcut_is_bit_exact(monkeypatch, mode, threshold):
    """OT(a, a) with the same tensors on both sides runs one soft-min per step (g copies f); passing
    clones forces the two-sided path. Both must agree bit for bit, and f must equal g."""
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
    set_mode(monkeypatch, mode)
    z = load_golden("solvers_small")
    x, a = dev(z["x"]), dev(z["a"])
    kw = dict(use_epsilon_scaling=False, eps=0.5, n_iters=25, threshold=threshold, check_every=4,
              return_prelast=True, return_n_iters=True)
    from flash_sinkhorn_b200 import _lib
    lib = _lib.load()
    c0 = lib.fs_launch_count()
    one = sinkhorn_flashstyle_symmetric(x, x.detach(), a, a.detach(), **kw)  # same memory, other objects
    c1 = lib.fs_launch_count()
    two = sinkhorn_flashstyle_symmetric(x, x.clone(), a, a.clone(), **kw)
    c2 = lib.fs_launch_count()
    assert c1 - c0 < c2 - c1  # the shortcut really ran fewer kernels
    assert one[4] == two[4]
    for u, v in zip(one[:4], two[:4]):
        assert torch.equal(u, v)
    assert torch.equal(one[0], one[1]) and torch.equal(one[2], one[3])
    want = O.solve_symmetric(z["x"].astype(np.float64), z["x"].astype(np.float64), z["a"].astype(np.float64),
                             z["a"].astype(np.float64), [0.5] * 25, threshold=threshold, check_every=4)
    assert rel(host(one[0]), want["f"]) < TOL[mode]


@pytest.mark.parametrize("name", ["full", "half"])
def test_implicit_gradient_vs_reference(monkeypatch, name):
    """implicit_grad_x_from_potentials on the CUDA engine (device-resident Schur CG) against the reference's
    result and the fp64 oracle; exact-fp32 products, as the reference defaults to."""
    from flash_sinkhorn_b200 import implicit_grad_x, implicit_grad_x_from_potentials
    set_mode(monkeypatch, "fp32")
    z = load_golden("implicit_small")
    x, y, a, b, gf, gg = (dev(z[k]) for k in ("x", "y", "a", "b", "grad_f", "grad_g"))
    fh, gh = dev(z[name + "_f_hat"]), dev(z[name + "_g_hat"])
    eps, cs = float(z[name + "_eps"]), float(z[name + "_cs"])
    gx, info = implicit_grad_x_from_potentials(x, y, fh, gh, gf, gg, eps=eps, log_a=a.log(), log_b=b.log(),
                                               cost_scale=cs, max_cg_iter=300)
    assert info.cg_converged and info.cg_iters <= int(z[name + "_cg"][1]) + 10
    assert rel(host(gx), z[name + "_grad_x"]) < 2e-3  # fp32 solves of a nearly singular system on both sides
    f64 = lambda k: z[k].astype(np.float64)
    want = O.implicit_grad_x(f64("x"), f64("y"), f64(name + "_f_hat"), f64(name + "_g_hat"), f64("grad_f"),
                             f64("grad_g"), np.log(f64("a")), np.log(f64("b")), eps, cost_scale=cs,
                             direct_solve=True)["grad_x"]
    assert rel(host(gx), want) < 2e-3
    # end-to-end wrapper: solves first, then differentiates (same potentials up to the solve's tolerance)
    gx2, info2 = implicit_grad_x(x, y, a, b, gf, gg, eps=eps, cost_scale=cs, n_iters=300, max_cg_iter=300)
    assert info2.cg_converged and rel(host(gx2), want) < 5e-3


def test_inverse_hvp_vs_reference(monkeypatch):
    from flash_sinkhorn_b200 import hvp_x_sqeuclid_from_potentials, inverse_hvp_x_sqeuclid_from_potentials
    set_mode(monkeypatch, "fp32")
    z = load_golden("implicit_small")
    x, y, gr, fo, go = (dev(z[k]) for k in ("inv_x", "inv_y", "inv_gr", "inv_f_ott", "inv_g_ott"))
    eps = float(z["inv_eps"])
    sol, info = inverse_hvp_x_sqeuclid_from_potentials(x, y, fo, go, gr, eps=eps, max_outer_iter=80,
                                                       max_inner_iter=300)
    assert info.cg_converged and info.cg_iters <= int(z["inv_cg"][1]) + 10
    assert rel(host(sol), z["inv_z"]) < 2e-3
    back, _ = hvp_x_sqeuclid_from_potentials(x, y, fo, go, sol, eps=eps, max_cg_iter=300, cg_rtol=1e-8, cg_atol=1e-8)
    assert rel(host(back), z["inv_gr"]) < 1e-4


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["unit", "mixed"])
def test_label_cost_vs_reference(monkeypatch, mode, name):
    """OTDD label-augmented cost (non-symmetric table, lambda_x != 1 in the 'mixed' case): solver, gradient
    kernel and SamplesLoss forward + grad_x, debiased and not, against the reference's results."""
    from flash_sinkhorn_b200 import SamplesLoss
    from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
    set_mode(monkeypatch, mode)
    z = load_golden("label_cost_small")
    x, y, a, b, W = (dev(z[k]) for k in ("x", "y", "a", "b", "W"))
    lx, ly = torch.as_tensor(z["label_x"]).cuda(), torch.as_tensor(z["label_y"]).cuda()
    lam_x, lam_y, cs, eps = (float(v) for v in z[name + "_lam"])
    kw = dict(label_x=lx, label_y=ly, label_cost_matrix=W, lambda_x=lam_x, lambda_y=lam_y)
    tol = TOL[mode]
    f, g, fp, gp = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=eps, n_iters=40,
                                                 cost_scale=cs, return_prelast=True, allow_tf32=(mode == "tf32"), **kw)
    for got, tag in ((f, "_f"), (g, "_g"), (fp, "_fpre"), (gp, "_gpre")):
        assert rel(host(got), z[name + tag]) < tol, tag
    gx, gy = sinkhorn_geomloss_online_grad_sqeuclid(x, y, a, b, dev(z[name + "_fpre"]), dev(z[name + "_gpre"]),
                                                    eps=eps, cost_scale=cs, allow_tf32=(mode == "tf32"), **kw)
    gtol = 3e-2 if mode == "tf32" else 3e-4
    assert rel(host(gx), z[name + "_grad_x"]) < gtol and rel(host(gy), z[name + "_grad_y"]) < gtol
    for debias, tag in ((False, "raw"), (True, "deb")):
        loss = SamplesLoss("sinkhorn", use_epsilon_scaling=False, eps=eps, n_iters=40, debias=debias,
                           half_cost=(cs == 0.5), allow_tf32=(mode == "tf32"), normalize=False,
                           label_cost_matrix=W, lambda_x=lam_x, lambda_y=lam_y)
        xr = x.clone().requires_grad_(True)
        val = loss(a, xr, b, y, label_x=lx, label_y=ly)
        (gxl,) = torch.autograd.grad(val, xr, create_graph=True)
        want = float(z[f"{name}_loss_{tag}"])
        assert abs(val.item() - want) < (2e-3 if mode == "tf32" else 5e-5) * max(1.0, abs(want))
        assert rel(host(gxl), z[f"{name}_loss_{tag}_grad_x"]) < gtol
        with pytest.raises(NotImplementedError):
            torch.autograd.grad(gxl.sum(), xr)  # HVP with a label cost, as in the reference
    with pytest.raises(ValueError):
        sinkhorn_flashstyle_symmetric(x, y, a, b, eps=eps, n_iters=3, use_epsilon_scaling=False,
                                      label_x=lx + 100, label_y=ly, label_cost_matrix=W, lambda_y=1.0)


def test_sharded_alternating_engine_on_a_one_rank_group():
    """The multi-GPU alternating path (half-steps through fs_symmetric_step_range + all-gather) on a one-rank
    NCCL group: against the reference fixtures and against the single-launch-sequence 1-GPU solver. The
    two-rank loop itself is covered on CPU (tests/test_sharded_gloo.py)."""
    import socket

    import torch.distributed as dist
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.distributed import alternating_solve_sharded
    from flash_sinkhorn_b200.kernels._common import log_weights
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    own_group = not dist.is_initialized()
    if own_group:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        z = load_golden("solvers_small")
        x, y, a, b, bn = (dev(z[k]) for k in ("x", "y", "a", "b", "b_normalised"))
        la, lb, lbn = log_weights(a).contiguous(), log_weights(b).contiguous(), log_weights(bn).contiguous()
        for prec, tol in ((_lib.PREC_SIMT, 2e-4), (_lib.PREC_FP32, 2e-4), (_lib.PREC_TF32, 2e-2)):
            for conv in (False, True):
                for rho in (None, 2.0):
                    f, g, k = alternating_solve_sharded(
                        x, y, la, lb, [0.4], 12, cost_scale=0.5, rho_x=rho, rho_y=rho, ott_convention=conv,
                        threshold=None, check_every=5, prec=prec, group=dist.group.WORLD)
                    tag = f"alt_{'ott' if conv else 'geo'}_{'bal' if rho is None else 'unb'}"
                    assert k == 12
                    assert rel(host(f), z[tag + "_f"]) < tol and rel(host(g), z[tag + "_g"]) < tol, (prec, tag)
        # early stop: same iteration count and potentials as the reference; annealed stages as the 1-GPU solver
        f, g, k = alternating_solve_sharded(x, y, la, lbn, [5.0], 80, cost_scale=1.0, rho_x=None, rho_y=None,
                                            ott_convention=False, threshold=1e-4, check_every=3,
                                            prec=_lib.PREC_FP32, group=dist.group.WORLD)
        assert k == int(z["alt_early_iters"]) and rel(host(f), z["alt_early_f"]) < 2e-4
        stages = [4.0, 2.0, 1.0, 0.5]
        f, g, k = alternating_solve_sharded(x, y, la, lb, stages, 5, cost_scale=1.0, rho_x=1.5, rho_y=None,
                                            ott_convention=False, threshold=None, check_every=5,
                                            prec=_lib.PREC_FP32, group=dist.group.WORLD)
        f1, g1, k1 = sinkhorn_flashstyle_alternating(x, y, a, b, n_iters=5, eps_list=stages, iters_per_eps=5,
                                                     rho_x=1.5, allow_tf32=False, return_n_iters=True)
        assert k == k1 == 20
        assert rel(host(f), host(f1)) < 1e-5 and rel(host(g), host(g1)) < 1e-5
        assert _lib.load().fs_device_error() == 0
    finally:
        if own_group:
            dist.destroy_process_group()
