"""Pins the CPU oracle (oracle/dense_sinkhorn.py) against fixtures produced by the reference itself
(tests/golden/make_golden.py). CPU only."""
import numpy as np
import pytest

from conftest import load_golden, rel_err
from oracle import dense_sinkhorn as O

F64 = np.float64


def d64(z, *names):
    return [z[k].astype(F64) for k in names]


def test_host_scalars():
    z = load_golden("solvers_small")
    x, y = z["x"], z["y"]
    assert abs(O.max_diameter(x, y) - float(z["diameter"])) < 1e-5 * float(z["diameter"])
    sched = O.epsilon_schedule(float(z["diameter"]), 0.3, 0.6)
    assert np.array_equal(np.array(sched, F64), z["sched"])  # bit-identical schedule
    assert O.dampening(0.5, None) == 1.0
    assert O.dampening(0.5, 2.0) == pytest.approx(1.0 / 1.25)
    lw = O.log_weights(np.array([0.5, 0.0, -1.0]))
    assert lw[1] == -100000.0 and lw[2] == -100000.0 and lw[0] == pytest.approx(np.log(0.5))


def test_single_kernels():
    z = load_golden("kernels_small")
    x, y, a, b, fh, gh = d64(z, "x", "y", "a", "b", "f_hat", "g_hat")
    eps, cs = float(z["eps"]), float(z["cost_scale"])
    la, lb = O.log_weights(a), O.log_weights(b)
    assert rel_err(O.lse_update(x, y, gh / eps + lb, eps, cs, 0.8), z["lse_raw"]) < 2e-5
    assert rel_err(O.lse_update_fused(x, y, gh, lb, eps, cs, 1.0), z["lse_fused"]) < 2e-5
    sf, sg = O.symmetric_step(x, y, fh, gh, la, lb, eps, cs, 0.5, 0.9, 0.7)
    assert rel_err(sf, z["step_f"]) < 2e-5 and rel_err(sg, z["step_g"]) < 2e-5
    vm, vn, mm, mn, sc = d64(z, "vec_m", "vec_n", "mat_m", "mat_n", "scale")
    assert rel_err(O.apply_vec(x, y, fh, gh, la, lb, vm, eps, 1, cs), z["apply_vec_axis1"]) < 1e-4
    assert rel_err(O.apply_vec(x, y, fh, gh, la, lb, vn, eps, 0, cs), z["apply_vec_axis0"]) < 1e-4
    assert rel_err(O.apply_mat(x, y, fh, gh, la, lb, mm, eps, 1, cs), z["apply_mat_axis1"]) < 1e-4
    assert rel_err(O.apply_mat(x, y, fh, gh, la, lb, mm, eps, 1, cs, scale=sc), z["apply_mat_axis1_scaled"]) < 1e-4
    assert rel_err(O.apply_mat(x, y, fh, gh, la, lb, mn, eps, 0, cs), z["apply_mat_axis0"]) < 1e-4
    f, g = d64(z, "f_std", "g_std")
    gx, gy = O.grad_xy(x, y, a, b, f, g, eps, cs, float(z["grad_scale"]))
    assert rel_err(gx, z["grad_x"]) < 1e-4 and rel_err(gy, z["grad_y"]) < 1e-4
    fo, go = d64(z, "f_ott", "g_ott")
    assert rel_err(O.mat5(x, y, fo, go, mn, eps, cs), z["mat5"]) < 1e-4


@pytest.mark.parametrize("name,cs,rx,ry", [("bal_sched", 1.0, None, None), ("half_semi", 0.5, 1.0, None),
                                           ("unbal", 1.0, 1.0, 4.0)])
def test_symmetric_solver(name, cs, rx, ry):
    z = load_golden("solvers_small")
    x, y, a, b = d64(z, "x", "y", "a", "b")
    s = O.solve_symmetric(x, y, a, b, list(z["sched"]), cost_scale=cs, rho_x=rx, rho_y=ry)
    for variant in ("fused", "sep"):
        tag = f"sym_{name}_{variant}"
        assert s["n_iters"] == int(z[tag + "_iters"])
        for k, key in (("f", "_f"), ("g", "_g"), ("f_pre", "_fpre"), ("g_pre", "_gpre")):
            assert rel_err(s[k], z[tag + key]) < 3e-5, (tag, k)


def test_symmetric_early_stop_and_warm_start():
    z = load_golden("solvers_small")
    x, y, a, b = d64(z, "x", "y", "a", "b_normalised")
    s = O.solve_symmetric(x, y, a, b, [5.0] * 60, threshold=1e-3, check_every=4)
    assert s["n_iters"] == int(z["sym_early_iters"]) < 62
    assert rel_err(s["f"], z["sym_early_f"]) < 3e-5 and rel_err(s["g"], z["sym_early_g"]) < 3e-5
    w = O.solve_symmetric(x, y, a, b, [5.0] * 3, last_extrapolation=False,
                          f_init=z["sym_early_f"].astype(F64), g_init=z["sym_early_g"].astype(F64))
    assert rel_err(w["f"], z["sym_warm_f"]) < 3e-5 and rel_err(w["g"], z["sym_warm_g"]) < 3e-5


@pytest.mark.parametrize("conv", [False, True])
@pytest.mark.parametrize("rho", [None, 2.0])
def test_alternating_solver(conv, rho):
    z = load_golden("solvers_small")
    x, y, a, b = d64(z, "x", "y", "a", "b")
    s = O.solve_alternating(x, y, a, b, [0.4], 12, cost_scale=0.5, rho_x=rho, rho_y=rho, ott_convention=conv)
    tag = f"alt_{'ott' if conv else 'geo'}_{'bal' if rho is None else 'unb'}"
    assert s["n_iters"] == int(z[tag + "_iters"]) == 12
    assert rel_err(s["f"], z[tag + "_f"]) < 3e-5 and rel_err(s["g"], z[tag + "_g"]) < 3e-5


def test_alternating_early_stop():
    z = load_golden("solvers_small")
    x, y, a, b = d64(z, "x", "y", "a", "b_normalised")
    s = O.solve_alternating(x, y, a, b, [5.0], 80, threshold=1e-4, check_every=3)
    assert s["n_iters"] == int(z["alt_early_iters"]) < 80
    assert rel_err(s["f"], z["alt_early_f"]) < 3e-5


def test_dense_reference_functions():
    z = load_golden("dense_reference")
    x, y, a, b = d64(z, "x", "y", "a", "b")
    diam = O.max_diameter(z["x"], z["y"])
    s = O.solve_symmetric(x, y, a, b, O.epsilon_schedule(diam, 0.4, 0.6))
    assert rel_err(s["f"], z["sym_f"]) < 3e-5 and rel_err(s["g"], z["sym_g"]) < 3e-5
    s = O.solve_symmetric(x, y, a, b, [0.3] * 20, last_extrapolation=False)
    assert rel_err(s["f"], z["fix_f"]) < 3e-5 and rel_err(s["g"], z["fix_g"]) < 3e-5
    gx, gy = O.grad_xy(x, y, a, b, z["fix_f"].astype(F64), z["fix_g"].astype(F64), 0.3)
    assert rel_err(gx, z["bary_gx"]) < 1e-4 and rel_err(gy, z["bary_gy"]) < 1e-4
    s = O.solve_alternating(x, y, a, b, [0.3], 15, ott_convention=True)
    assert rel_err(s["f"], z["ott_f"]) < 3e-5 and rel_err(s["g"], z["ott_g"]) < 3e-5


LOSS_CASES = {
    "bal_debias_half": dict(blur=0.5, scaling=0.7, debias=True, cost_scale=0.5),
    "bal_fixed": dict(eps_list=[0.36] * 25),
    "semi": dict(blur=0.5, scaling=0.7, rho_x=1.5**2),
    "unbal": dict(blur=0.5, scaling=0.7, rho_x=1.2**2, rho_y=1.2**2),
}


@pytest.mark.parametrize("name", sorted(LOSS_CASES))
def test_samples_loss(name):
    z = load_golden("samples_loss_small")
    x, y, a, b = d64(z, "x", "y", "a", "b")
    cfg = dict(LOSS_CASES[name])
    if "eps_list" in cfg:
        sched = cfg.pop("eps_list")
    else:
        sched = O.epsilon_schedule(O.max_diameter(z["x"], z["y"]), cfg.pop("blur"), cfg.pop("scaling"))
    r = O.samples_loss(x, y, a, b, sched, want_grad_x=True, **cfg)
    assert abs(r["loss"] - float(z[name + "_loss"])) < 2e-5 * max(1.0, abs(float(z[name + "_loss"])))
    assert rel_err(r["grad_x"], z[name + "_gx"]) < 2e-4


def test_samples_loss_alternating_and_uniform():
    z = load_golden("samples_loss_small")
    x, y, a, b = d64(z, "x", "y", "a", "b")
    s = O.solve_alternating(x, y, a, b, [0.3], 15)
    assert rel_err(s["f"], z["alt_f"]) < 3e-5
    assert abs(O.ot_cost(a, b, s["f"], s["g"], 0.3) - float(z["alt_loss"])) < 2e-5 * abs(float(z["alt_loss"]))
    n, m = x.shape[0], y.shape[0]
    sched = O.epsilon_schedule(O.max_diameter(z["x"], z["y"]), 0.5, 0.7)
    r = O.samples_loss(x, y, np.full(n, 1.0 / n), np.full(m, 1.0 / m), sched)
    # weights created in fp32 by the reference (1/n rounded): tolerance covers that
    assert abs(r["loss"] - float(z["xy_loss"])) < 1e-5 * abs(float(z["xy_loss"]))


@pytest.mark.parametrize("name,rx,ry,cs", [("bal", None, None, 1.0), ("semi_half", 2.0, None, 0.5)])
def test_hvp(name, rx, ry, cs):
    z = load_golden("hvp_small")
    x, y, A, fo, go = d64(z, "x", "y", "A", name + "_f_ott", name + "_g_ott")
    eps = float(z["eps"])
    r = O.hvp_x(x, y, fo, go, A, eps, rho_x=rx, rho_y=ry, cost_scale=cs, max_cg_iter=400)
    assert rel_err(r["hvp"], z[name + "_hvp"]) < 3e-4
    if name + "_hvp_dense" in z:
        assert rel_err(r["hvp"], z[name + "_hvp_dense"]) < 1e-4
    direct = O.hvp_x(x, y, fo, go, A, eps, rho_x=rx, rho_y=ry, cost_scale=cs, direct_solve=True)
    assert rel_err(direct["hvp"], r["hvp"]) < 1e-3


def test_config1_golden_is_recorded():
    z = load_golden("config1")
    # Values measured independently on the fp32 dense path of the reference.
    assert float(z["loss"]) == pytest.approx(36.8802109, rel=2e-6)
    assert float(z["grad_x_norm"]) == pytest.approx(0.128287598, rel=2e-4)


@pytest.mark.parametrize("name", ["full", "half"])
def test_implicit_gradient(name):
    """Oracle vs the reference's implicit_grad_x_from_potentials (CG and direct solve of the Schur system)."""
    z = load_golden("implicit_small")
    x, y, a, b, gf, gg = d64(z, "x", "y", "a", "b", "grad_f", "grad_g")
    fh, gh = d64(z, name + "_f_hat", name + "_g_hat")
    eps, cs = float(z[name + "_eps"]), float(z[name + "_cs"])
    want = z[name + "_grad_x"].astype(F64)
    conv, iters, _ = z[name + "_cg"]
    assert conv == 1.0
    got = O.implicit_grad_x(x, y, fh, gh, gf, gg, np.log(a), np.log(b), eps, cost_scale=cs, max_cg_iter=300)
    # the reference iterates in fp32, the oracle in fp64: it may need fewer steps, never noticeably more
    assert got["cg_converged"] and got["cg_iters"] <= int(iters) + 3
    # the Schur system is nearly singular along constants (only tau2 = 1e-5 regularises it), so the
    # reference's fp32 solve carries ~5e-4 of error relative to this fp64 restatement
    assert rel_err(got["grad_x"], want) < 2e-3
    direct = O.implicit_grad_x(x, y, fh, gh, gf, gg, np.log(a), np.log(b), eps, cost_scale=cs, direct_solve=True)
    assert rel_err(direct["grad_x"], want) < 2e-3
    assert rel_err(direct["grad_x"], got["grad_x"]) < 1e-4


def test_inverse_hvp():
    """Oracle vs the reference's inverse_hvp_x_sqeuclid_from_potentials (positive definite case, eps = 5)."""
    z = load_golden("implicit_small")
    x, y, gr, fo, go = d64(z, "inv_x", "inv_y", "inv_gr", "inv_f_ott", "inv_g_ott")
    eps = float(z["inv_eps"])
    conv, iters, res, res0 = z["inv_cg"]
    assert conv == 1.0 and res <= 1e-6 * res0 + 1e-6
    want = z["inv_z"].astype(F64)
    got = O.inverse_hvp_x(x, y, fo, go, gr, eps, max_outer_iter=80)
    assert got["cg_converged"] and got["cg_iters"] <= int(iters) + 3
    assert rel_err(got["z"], want) < 5e-4
    direct = O.inverse_hvp_x(x, y, fo, go, gr, eps, direct_solve=True)
    assert rel_err(direct["z"], want) < 5e-4
    # H z reproduces the right-hand side
    back = O.hvp_x(x, y, fo, go, direct["z"], eps, direct_solve=True)["hvp"]
    assert rel_err(back, gr) < 1e-8


@pytest.mark.parametrize("name", ["a", "b"])
def test_c_transform(name):
    """Oracle vs the reference's c_transform_fwd / c_transform_cost (values, indices, Danskin gradients)."""
    z = load_golden("c_transform_small")
    x, y, psi, wa, wb = d64(z, name + "_x", name + "_y", name + "_psi", name + "_wa", name + "_wb")
    cs = float(z[name + "_cs"])
    c, idx = O.c_transform(x, y, psi, cs)
    assert np.array_equal(idx, z[name + "_idx"])
    assert np.abs(c - z[name + "_c"]).max() < 1e-4
    r = O.c_transform_cost(x, y, psi, wa, wb, cs)
    assert abs(r["loss"] - float(z[name + "_loss"])) < 1e-5 * max(1.0, abs(float(z[name + "_loss"])))
    assert rel_err(r["grad_x"], z[name + "_grad_x"]) < 1e-5
    assert np.abs(r["grad_psi"] - z[name + "_grad_psi"]).max() < 1e-6


def test_c_transform_tie_break():
    z = load_golden("c_transform_small")
    y = z["tie_y"].astype(F64)
    _, idx = O.c_transform(np.zeros((1, 4)), y, np.zeros(96))
    assert int(z["tie_idx"][0]) == 0 and int(idx[0]) == 0  # equidistant targets 0 and 64: the smaller index


@pytest.mark.parametrize("name", ["unit", "mixed"])
def test_label_cost(name):
    """Oracle vs the reference's label-augmented symmetric solve, gradient kernel and SamplesLoss."""
    z = load_golden("label_cost_small")
    x, y, a, b, W = d64(z, "x", "y", "a", "b", "W")
    lx, ly = z["label_x"], z["label_y"]
    lam_x, lam_y, cs, eps = (float(v) for v in z[name + "_lam"])
    kw = dict(lambda_x=lam_x, lambda_y=lam_y, cost_scale=cs)
    s = O.label_solve_symmetric(x, y, a, b, [eps] * 40, lx, ly, W, **kw)
    for key, tag in (("f", "_f"), ("g", "_g"), ("f_pre", "_fpre"), ("g_pre", "_gpre")):
        assert np.isfinite(z[name + tag]).all()
        assert rel_err(s[key], z[name + tag]) < 3e-5, key
    gx, gy = O.label_grad_xy(x, y, a, b, z[name + "_fpre"].astype(F64), z[name + "_gpre"].astype(F64), eps, lx, ly,
                             W, **kw)
    assert rel_err(gx, z[name + "_grad_x"]) < 1e-4 and rel_err(gy, z[name + "_grad_y"]) < 1e-4
    for debias, tag in ((False, "raw"), (True, "deb")):
        r = O.label_samples_loss(x, y, a, b, [eps] * 40, lx, ly, W, debias=debias, **kw)
        want = float(z[f"{name}_loss_{tag}"])
        assert abs(r["loss"] - want) < 2e-5 * max(1.0, abs(want)), (debias, r["loss"], want)
        assert rel_err(r["grad_x"], z[f"{name}_loss_{tag}_grad_x"]) < 2e-4


def test_legacy_ott_surface():
    """Signed log-sum-exp, OTT-convention half-steps, solve and plan applications: the oracle against the
    reference's Triton kernels (interpreter) and against its dense functions."""
    z = load_golden("legacy_ott_small")
    x, y, f, g, vm, vn = d64(z, "x", "y", "f", "g", "vec_m", "vec_n")
    eps = float(z["eps"])
    for axis, vec in ((1, vm), (0, vn)):
        out, sgn = O.signed_lse_ott(x, y, f, g, eps, axis)
        assert rel_err(out, z[f"lse_axis{axis}"]) < 2e-5 and np.all(sgn == 1.0)
        assert np.all(z[f"lse_sgn_axis{axis}"] == 1.0)
        out, sgn = O.signed_lse_ott(x, y, f, g, eps, axis, vec=vec)
        # log|sum| is ill-conditioned where positive and negative parts nearly cancel: absolute tolerance
        assert np.abs(out - z[f"vlse_axis{axis}"]).max() < 5e-4
        assert np.abs(out - z[f"vlse_dense_axis{axis}"]).max() < 5e-4
        assert np.array_equal(sgn, z[f"vlse_sgn_axis{axis}"]) and np.array_equal(sgn, z[f"vlse_dense_sgn_axis{axis}"])
    out, sgn = O.signed_lse_ott(x, y, f, g, eps, 1, vec=np.zeros_like(vm))
    assert np.all(np.isneginf(out)) and np.all(sgn == 0)
    assert np.all(np.isneginf(z["zero_vec_lse"])) and np.all(z["zero_vec_sgn"] == 0)

    la, lb = d64(z, "loga", "logb")
    assert rel_err(O.update_potential_ott(x, y, f, g, lb, eps, 0), z["update_g"]) < 2e-5
    assert rel_err(O.update_potential_ott(x, y, f, g, lb, eps, 0), z["update_g_dense"]) < 2e-5
    assert rel_err(O.update_potential_ott(x, y, f, g, la, eps, 1), z["update_f"]) < 2e-5
    fo, go = O.sinkhorn_potentials_ott(x, y, la, lb, eps, 6)
    assert rel_err(fo, z["ott_f_dense"]) < 2e-5 and rel_err(go, z["ott_g_dense"]) < 2e-5
    assert rel_err(fo, z["ott_f_facade"]) < 2e-5 and rel_err(go, z["ott_g_facade"]) < 2e-5
    # the facade is the alternating solver in OTT convention
    alt = O.solve_alternating(x, y, np.exp(la), np.exp(lb), [eps], 6, ott_convention=True)
    assert rel_err(alt["f"], z["ott_f_facade"]) < 2e-5 and rel_err(alt["g"], z["ott_g_facade"]) < 2e-5
    assert rel_err(O.apply_transport_ott(x, y, fo, go, vm, eps, 1), z["transport_axis1"]) < 1e-4
    assert rel_err(O.apply_transport_ott(x, y, fo, go, vm, eps, 1), z["transport_dense_axis1"]) < 1e-4
    assert rel_err(O.apply_transport_ott(x, y, fo, go, vn, eps, 0), z["transport_axis0"]) < 1e-4

    # deprecated OTT-convention plan applications == products with the dense OTT plan
    cs = float(z["cs"])
    fh, gh, mm, mn, sc = d64(z, "cs_f", "cs_g", "mat_m", "mat_n", "scale")
    P = O.plan_ott(x, y, fh, gh, eps, cs)
    assert rel_err(P @ vm, z["dep_vec_axis1"]) < 1e-4
    assert rel_err(P.T @ vn, z["dep_vec_axis0"]) < 1e-4
    assert rel_err(P @ (mm * sc[:, None]), z["dep_mat_axis1"]) < 1e-4
    assert rel_err(P.T @ mn, z["dep_mat_axis0"]) < 1e-4
