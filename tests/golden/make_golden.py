"""Generate the golden fixtures under tests/golden/ by running the REFERENCE itself.

Run once, in a container that has the reference checkout (no GPU needed):

    TRITON_INTERPRET=1 PYTHONPATH=<reference>/src python tests/golden/make_golden.py [--skip-c1]

Two sources of truth are used:
  * the reference's dense PyTorch oracles (testing/reference_sinkhorn.py,
    testing/reference_hvp.py), on CPU tensors;
  * the reference's own Triton kernels and host loops (SamplesLoss, solvers, apply,
    gradient, mat5, HVP) executed on CPU tensors by the Triton interpreter. The library
    refuses non-CUDA tensors in a few wrappers, so ``torch.Tensor.is_cuda`` is patched to
    report True for the duration of this script; no reference source is modified.

Inputs are drawn from a CPU ``torch.Generator`` and stored next to the outputs, so the
tests never need the reference. Everything is float32 unless noted.
"""
import argparse
import math
import os
import sys
import time

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

torch.Tensor.is_cuda = property(lambda self: True)  # see module docstring

import flash_sinkhorn  # noqa: E402  (the reference)
from flash_sinkhorn import SamplesLoss  # noqa: E402
from flash_sinkhorn.hvp import geomloss_to_ott_potentials, hvp_x_sqeuclid_from_potentials  # noqa: E402
from flash_sinkhorn.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle  # noqa: E402
from flash_sinkhorn.kernels.apply_ott import mat5_sqeuclid  # noqa: E402
from flash_sinkhorn.kernels.sinkhorn_flashstyle_sqeuclid import (  # noqa: E402
    flashsinkhorn_lse,
    flashsinkhorn_lse_fused,
    flashsinkhorn_symmetric_step,
)
from flash_sinkhorn.kernels.sinkhorn_triton_grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid  # noqa: E402
from flash_sinkhorn.kernels._common import epsilon_schedule, log_weights, max_diameter  # noqa: E402
from flash_sinkhorn.sinkhorn_solvers import sinkhorn_flashstyle_alternating, sinkhorn_flashstyle_symmetric  # noqa: E402
from flash_sinkhorn.testing import reference_hvp, reference_sinkhorn  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
MANUAL = dict(autotune=False, block_m=32, block_n=32, block_k=16)  # the autotuner needs a GPU driver


def np32(t):
    return t.detach().cpu().numpy().astype(np.float32)


def clouds(seed, n, m, d, shift=0.0, weights="uniform", mass_b=1.0):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n, d, generator=gen)
    y = shift + torch.randn(m, d, generator=gen)
    if weights == "uniform":
        a = torch.full((n,), 1.0 / n)
        b = torch.full((m,), mass_b / m)
    else:
        a = torch.softmax(torch.randn(n, generator=gen), dim=0)
        b = torch.softmax(torch.randn(m, generator=gen), dim=0) * mass_b
    return x, y, a, b


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"wrote {path} ({os.path.getsize(path)} bytes)")


def gen_kernels():
    """Single kernel calls: LSE (raw/fused bias), symmetric step, apply vec/mat, gradient, mat5."""
    n, m, d = 70, 52, 12
    x, y, a, b = clouds(11, n, m, d, shift=0.3, weights="softmax", mass_b=1.3)
    eps, cs = 0.37, 0.5
    gen = torch.Generator().manual_seed(12)
    f_hat = -cs * (x**2).sum(1) + 0.1 * torch.randn(n, generator=gen)
    g_hat = -cs * (y**2).sum(1) + 0.1 * torch.randn(m, generator=gen)
    la, lb = log_weights(a), log_weights(b)
    bias = g_hat / eps + lb
    out = dict(x=np32(x), y=np32(y), a=np32(a), b=np32(b), f_hat=np32(f_hat), g_hat=np32(g_hat),
               eps=np.float64(eps), cost_scale=np.float64(cs))
    kw = dict(allow_tf32=False, **MANUAL)
    out["lse_raw"] = np32(flashsinkhorn_lse(x, y, bias, eps, cost_scale=cs, damping=0.8, **kw))
    out["lse_fused"] = np32(flashsinkhorn_lse_fused(x, y, g_hat, lb, eps, cost_scale=cs, damping=1.0, **kw))
    fs, gs = flashsinkhorn_symmetric_step(x, y, f_hat, g_hat, la, lb, eps, cost_scale=cs, alpha=0.5,
                                          damping_f=0.9, damping_g=0.7, **kw)
    out["step_f"], out["step_g"] = np32(fs), np32(gs)
    vec_m = torch.randn(m, generator=gen)
    vec_n = torch.randn(n, generator=gen)
    akw = dict(eps=eps, cost_scale=cs, allow_tf32=False)
    out["vec_m"], out["vec_n"] = np32(vec_m), np32(vec_n)
    out["apply_vec_axis1"] = np32(apply_plan_vec_flashstyle(x, y, f_hat, g_hat, la, lb, vec_m, axis=1,
                                                            block_m=32, block_n=32, block_k=16, **akw))
    out["apply_vec_axis0"] = np32(apply_plan_vec_flashstyle(x, y, f_hat, g_hat, la, lb, vec_n, axis=0,
                                                            block_m=32, block_n=32, block_k=16, **akw))
    mat_m = torch.randn(m, d, generator=gen)
    mat_n = torch.randn(n, d, generator=gen)
    scale = torch.randn(m, generator=gen)
    out["mat_m"], out["mat_n"], out["scale"] = np32(mat_m), np32(mat_n), np32(scale)
    mkw = dict(block_d=16, **MANUAL)
    out["apply_mat_axis1"] = np32(apply_plan_mat_flashstyle(x, y, f_hat, g_hat, la, lb, mat_m, axis=1, **akw, **mkw))
    out["apply_mat_axis1_scaled"] = np32(apply_plan_mat_flashstyle(x, y, f_hat, g_hat, la, lb, mat_m, axis=1,
                                                                   scale=scale, **akw, **mkw))
    out["apply_mat_axis0"] = np32(apply_plan_mat_flashstyle(x, y, f_hat, g_hat, la, lb, mat_n, axis=0, **akw, **mkw))
    # gradient kernel from standard potentials
    f_std = f_hat + cs * (x**2).sum(1)
    g_std = g_hat + cs * (y**2).sum(1)
    gsc = torch.tensor(1.7)
    gx, gy = sinkhorn_geomloss_online_grad_sqeuclid(x, y, a, b, f_std, g_std, eps=eps, allow_tf32=False,
                                                    cost_scale=cs, grad_scale=gsc, num_warps=4, **MANUAL)
    out["f_std"], out["g_std"], out["grad_scale"] = np32(f_std), np32(g_std), np.float32(1.7)
    out["grad_x"], out["grad_y"] = np32(gx), np32(gy)
    # mat5 with OTT-convention potentials
    f_ott, g_ott = geomloss_to_ott_potentials(f_std, g_std, a, b, eps=eps)
    out["f_ott"], out["g_ott"] = np32(f_ott), np32(g_ott)
    out["mat5"] = np32(mat5_sqeuclid(x, y, f_ott, g_ott, mat_n, eps=eps, cost_scale=cs, allow_tf32=False, **MANUAL))
    save("kernels_small", **out)


def gen_solvers():
    """Whole solves through the reference's host loops + Triton kernels (interpreter)."""
    n, m, d = 96, 80, 16
    x, y, a, b = clouds(21, n, m, d, shift=0.2, weights="softmax", mass_b=1.3)
    base = dict(x=np32(x), y=np32(y), a=np32(a), b=np32(b))
    out = dict(base)
    cases = {
        "bal_sched": dict(cost_scale=1.0, rho_x=None, rho_y=None),
        "half_semi": dict(cost_scale=0.5, rho_x=1.0, rho_y=None),
        "unbal": dict(cost_scale=1.0, rho_x=1.0, rho_y=4.0),
    }
    diam = max_diameter(x, y)
    sched = epsilon_schedule(diam, 0.3, 0.6, p=2.0)
    out["sched"] = np.array(sched, np.float64)
    out["diameter"] = np.float64(diam)
    for name, c in cases.items():
        for fused in (True, False):
            f, g, fp, gp, k = sinkhorn_flashstyle_symmetric(
                x, y, a, b, blur=0.3, scaling=0.6, use_epsilon_scaling=True, allow_tf32=False, autotune=False,
                fused=fused, return_prelast=True, return_n_iters=True, **c)
            tag = f"sym_{name}_{'fused' if fused else 'sep'}"
            out[tag + "_f"], out[tag + "_g"] = np32(f), np32(g)
            out[tag + "_fpre"], out[tag + "_gpre"] = np32(fp), np32(gp)
            out[tag + "_iters"] = np.int64(k)
    # fixed eps + early stopping (equal masses, otherwise the balanced iteration drifts and never stops)
    bn = b / b.sum()
    out["b_normalised"] = np32(bn)
    f, g, k = sinkhorn_flashstyle_symmetric(x, y, a, bn, use_epsilon_scaling=False, eps=5.0, n_iters=60,
                                            allow_tf32=False, autotune=False, threshold=1e-3, check_every=4,
                                            return_n_iters=True)
    out["sym_early_f"], out["sym_early_g"], out["sym_early_iters"] = np32(f), np32(g), np.int64(k)
    # warm start
    f2, g2 = sinkhorn_flashstyle_symmetric(x, y, a, bn, use_epsilon_scaling=False, eps=5.0, n_iters=3,
                                           allow_tf32=False, autotune=False, f_init=f, g_init=g,
                                           last_extrapolation=False)
    out["sym_warm_f"], out["sym_warm_g"] = np32(f2), np32(g2)
    # alternating
    for conv in (False, True):
        for rho in (None, 2.0):
            f, g, k = sinkhorn_flashstyle_alternating(x, y, a, b, eps=0.4, n_iters=12, cost_scale=0.5,
                                                      rho_x=rho, rho_y=rho, allow_tf32=False, autotune=False,
                                                      ott_convention=conv, return_n_iters=True)
            tag = f"alt_{'ott' if conv else 'geo'}_{'bal' if rho is None else 'unb'}"
            out[tag + "_f"], out[tag + "_g"], out[tag + "_iters"] = np32(f), np32(g), np.int64(k)
    f, g, k = sinkhorn_flashstyle_alternating(x, y, a, bn, eps=5.0, n_iters=80, allow_tf32=False, autotune=False,
                                              threshold=1e-4, check_every=3, return_n_iters=True)
    out["alt_early_f"], out["alt_early_g"], out["alt_early_iters"] = np32(f), np32(g), np.int64(k)
    save("solvers_small", **out)


def gen_samples_loss():
    """SamplesLoss forward / backward / double backward through the reference's autograd glue."""
    n, m, d = 64, 48, 8
    x, y, a, b = clouds(31, n, m, d, shift=0.25, weights="softmax", mass_b=1.0)
    out = dict(x=np32(x), y=np32(y), a=np32(a), b=np32(b))
    gen = torch.Generator().manual_seed(32)
    v = torch.randn(n, d, generator=gen)
    out["v"] = np32(v)
    common = dict(allow_tf32=False, autotune=False, block_m=32, block_n=32, block_k=16)
    configs = {
        "bal_debias_half": dict(blur=0.5, scaling=0.7, debias=True, half_cost=True),
        "bal_fixed": dict(blur=0.6, use_epsilon_scaling=False, eps=0.36, n_iters=25),
        "semi": dict(blur=0.5, scaling=0.7, reach_x=1.5),
        "unbal": dict(blur=0.5, scaling=0.7, reach=1.2, normalize=False),
        "alt": dict(backend="alternating", use_epsilon_scaling=False, eps=0.3, n_iters=15, blur=0.5),
    }
    for name, cfg in configs.items():
        xs = x.clone().requires_grad_(True)
        ys = y.clone().requires_grad_(True)
        a_s = a.clone().requires_grad_(True)
        loss_fn = SamplesLoss("sinkhorn", **cfg, **common)
        val = loss_fn(a_s, xs, b, ys)
        gx, gy, ga = torch.autograd.grad(val, (xs, ys, a_s))
        out[name + "_loss"] = np.float32(val.item())
        out[name + "_gx"], out[name + "_gy"], out[name + "_ga"] = np32(gx), np32(gy), np32(ga)
        f, g = SamplesLoss("sinkhorn", potentials=True, **cfg, **common)(a, x, b, y)
        out[name + "_f"], out[name + "_g"] = np32(f), np32(g)
    # (x, y) call form with uniform weights
    out["xy_loss"] = np.float32(SamplesLoss("sinkhorn", blur=0.5, scaling=0.7, **common)(x, y).item())
    save("samples_loss_small", **out)


def gen_hvp():
    """HVP: reference streaming implementation (interpreter) and its dense oracle."""
    n, m, d = 40, 32, 6
    x, y, a, b = clouds(41, n, m, d, shift=0.2, weights="softmax", mass_b=1.0)
    gen = torch.Generator().manual_seed(42)
    A = torch.randn(n, d, generator=gen)
    eps = 0.45
    out = dict(x=np32(x), y=np32(y), a=np32(a), b=np32(b), A=np32(A), eps=np.float64(eps))
    for name, (rx, ry, cs) in {"bal": (None, None, 1.0), "semi_half": (2.0, None, 0.5)}.items():
        f, g, fp, gp = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=eps, n_iters=200,
                                                     allow_tf32=False, autotune=False, return_prelast=True,
                                                     cost_scale=cs, rho_x=rx, rho_y=ry)
        f_ott, g_ott = geomloss_to_ott_potentials(fp, gp, a, b, eps=eps)
        hv, info = hvp_x_sqeuclid_from_potentials(x, y, f_ott, g_ott, A, eps=eps, rho_x=rx, rho_y=ry, cost_scale=cs,
                                                  max_cg_iter=400, autotune=False, block_m=32, block_n=32, block_k=16)
        out[name + "_f_ott"], out[name + "_g_ott"] = np32(f_ott), np32(g_ott)
        out[name + "_hvp"] = np32(hv)
        out[name + "_cg"] = np.array([float(info.cg_converged), info.cg_iters, info.cg_residual,
                                      info.cg_initial_residual], np.float64)
        if cs == 1.0:
            dense, _ = reference_hvp.hvp_x_dense_sqeuclid_semi_unbalanced(
                x, y, f_ott, g_ott, A, eps=eps, rho_x=rx, rho_y=ry, max_cg_iter=400,
                use_preconditioner=False)  # its default Neumann preconditioner diverges on this case
            out[name + "_hvp_dense"] = np32(dense)
    save("hvp_small", **out)


def gen_implicit():
    """Implicit gradient (implicit_grad.py) and inverse HVP (hvp.py:696-835) of the reference, interpreter run.
    The autotuned kernels cannot run without a GPU driver and these two wrappers do not forward
    ``autotune``; the module-level names they call are therefore wrapped with ``autotune=False`` for the
    run (functools.partial on the imported functions; no reference source is modified)."""
    import functools

    import flash_sinkhorn.hvp as ref_hvp
    import flash_sinkhorn.implicit_grad as ref_ig

    ref_ig.apply_plan_mat_flashstyle = functools.partial(ref_ig.apply_plan_mat_flashstyle, **MANUAL)
    ref_hvp.hvp_x_sqeuclid_from_potentials = functools.partial(ref_hvp.hvp_x_sqeuclid_from_potentials,
                                                               autotune=False)
    n, m, d = 40, 32, 6
    x, y, a, b = clouds(61, n, m, d, shift=0.2, weights="softmax")
    gen = torch.Generator().manual_seed(62)
    grad_f, grad_g = torch.randn(n, generator=gen), torch.randn(m, generator=gen)
    out = dict(x=np32(x), y=np32(y), a=np32(a), b=np32(b), grad_f=np32(grad_f), grad_g=np32(grad_g))
    for name, (eps, cs) in {"full": (0.45, 1.0), "half": (0.3, 0.5)}.items():
        f, g = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=eps, n_iters=300,
                                             allow_tf32=False, autotune=False, cost_scale=cs)
        f_hat, g_hat = f - cs * (x**2).sum(1), g - cs * (y**2).sum(1)
        gx, info = ref_ig.implicit_grad_x_from_potentials(x, y, f_hat, g_hat, grad_f, grad_g, eps=eps,
                                                          log_a=a.log(), log_b=b.log(), cost_scale=cs,
                                                          max_cg_iter=300)
        out[name + "_eps"], out[name + "_cs"] = np.float64(eps), np.float64(cs)
        out[name + "_f_hat"], out[name + "_g_hat"] = np32(f_hat), np32(g_hat)
        out[name + "_grad_x"] = np32(gx)
        out[name + "_cg"] = np.array([float(info.cg_converged), info.cg_iters, info.cg_residual], np.float64)
    # inverse HVP where the Hessian is positive definite (large eps); small problem: every outer CG
    # iteration is a full HVP with its own inner solve under the interpreter
    n, m, d = 24, 20, 3
    x, y, a, b = clouds(63, n, m, d, shift=0.2, weights="softmax")
    gr = torch.randn(n, d, generator=torch.Generator().manual_seed(64))
    eps = 5.0
    f, g, fp, gp = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=eps, n_iters=200,
                                                 allow_tf32=False, autotune=False, return_prelast=True)
    f_ott, g_ott = geomloss_to_ott_potentials(fp, gp, a, b, eps=eps)
    z, info = ref_hvp.inverse_hvp_x_sqeuclid_from_potentials(x, y, f_ott, g_ott, gr, eps=eps, max_outer_iter=80,
                                                             max_inner_iter=300, block_m=32, block_n=32, block_k=16)
    out.update(inv_x=np32(x), inv_y=np32(y), inv_a=np32(a), inv_b=np32(b), inv_gr=np32(gr),
               inv_eps=np.float64(eps), inv_f_ott=np32(f_ott), inv_g_ott=np32(g_ott), inv_z=np32(z),
               inv_cg=np.array([float(info.cg_converged), info.cg_iters, info.cg_residual,
                                info.cg_initial_residual], np.float64))
    save("implicit_small", **out)


def gen_label_cost():
    """OTDD label-augmented cost: the reference's symmetric solver, gradient kernel and SamplesLoss
    (forward + grad_x, debiased and not) with a non-symmetric label table, interpreter run."""
    n, m, d, V = 60, 44, 7, 5
    x, y, a, b = clouds(81, n, m, d, shift=0.25, weights="softmax")
    gen = torch.Generator().manual_seed(82)
    lx = torch.randint(0, V, (n,), generator=gen)
    ly = torch.randint(0, V, (m,), generator=gen)
    W = torch.rand(V, V, generator=gen) * 2.0
    W.fill_diagonal_(0.0)
    out = dict(x=np32(x), y=np32(y), a=np32(a), b=np32(b), label_x=lx.numpy().astype(np.int64),
               label_y=ly.numpy().astype(np.int64), W=np32(W))
    for name, (lam_x, lam_y, cs, eps) in {"unit": (1.0, 1.0, 1.0, 0.5), "mixed": (0.7, 1.8, 0.5, 0.4)}.items():
        kw = dict(label_x=lx, label_y=ly, label_cost_matrix=W, lambda_x=lam_x, lambda_y=lam_y)
        f, g, fp, gp = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=eps, n_iters=40,
                                                     allow_tf32=False, autotune=False, cost_scale=cs,
                                                     return_prelast=True, **kw)
        gx, gy = sinkhorn_geomloss_online_grad_sqeuclid(x, y, a, b, fp, gp, eps=eps, allow_tf32=False, cost_scale=cs,
                                                        num_warps=4, **MANUAL, **kw)
        out.update({name + "_lam": np.array([lam_x, lam_y, cs, eps], np.float64), name + "_f": np32(f),
                    name + "_g": np32(g), name + "_fpre": np32(fp), name + "_gpre": np32(gp),
                    name + "_grad_x": np32(gx), name + "_grad_y": np32(gy)})
        for debias in (False, True):
            loss = SamplesLoss("sinkhorn", use_epsilon_scaling=False, eps=eps, n_iters=40, debias=debias,
                               half_cost=(cs == 0.5), allow_tf32=False, autotune=False, normalize=False,
                               label_cost_matrix=W, lambda_x=lam_x, lambda_y=lam_y)
            xr = x.clone().requires_grad_(True)
            val = loss(a, xr, b, y, label_x=lx, label_y=ly)
            (gxl,) = torch.autograd.grad(val, xr)
            tag = f"{name}_loss_{'deb' if debias else 'raw'}"
            out[tag], out[tag + "_grad_x"] = np.float64(val.item()), np32(gxl)
    save("label_cost_small", **out)


def gen_c_transform():
    """Hard c-transform (c_transform.py, kernels/c_transform_sqeuclid.py), interpreter run with manual blocks:
    values, arg-min indices, the semi-dual objective and its Danskin gradients; plus the tie-break case of
    the reference's test_c_transform.py:179-212 (two equidistant targets in different tiles)."""
    from flash_sinkhorn.c_transform import c_transform_cost, c_transform_fwd

    man = dict(autotune=False, block_m=32, block_n=32, block_k=16)
    out = {}
    for name, (n, m, d, cs) in {"a": (90, 130, 5, 1.0), "b": (150, 70, 24, 0.5)}.items():
        gen = torch.Generator().manual_seed(71 + n)
        x, y, psi = torch.randn(n, d, generator=gen), torch.randn(m, d, generator=gen), torch.randn(m, generator=gen)
        wa = torch.softmax(torch.randn(n, generator=gen), 0)
        wb = torch.softmax(torch.randn(m, generator=gen), 0)
        c, idx = c_transform_fwd(x, y, psi, cost_scale=cs, allow_tf32=False, **man)
        xr, pr = x.clone().requires_grad_(True), psi.clone().requires_grad_(True)
        # c_transform_cost does not forward block sizes: wrap the kernel it calls for the run
        import functools

        import flash_sinkhorn.c_transform as ref_ct
        orig = ref_ct.c_transform_kernel
        ref_ct.c_transform_kernel = functools.partial(orig, block_m=32, block_n=32, block_k=16)
        try:
            loss = c_transform_cost(xr, y, pr, cost_scale=cs, allow_tf32=False, autotune=False, a=wa, b=wb)
        finally:
            ref_ct.c_transform_kernel = orig
        gx, gpsi = torch.autograd.grad(loss, [xr, pr])
        out.update({name + "_x": np32(x), name + "_y": np32(y), name + "_psi": np32(psi), name + "_wa": np32(wa),
                    name + "_wb": np32(wb), name + "_cs": np.float64(cs), name + "_c": np32(c),
                    name + "_idx": idx.numpy().astype(np.int64), name + "_loss": np.float64(loss.item()),
                    name + "_grad_x": np32(gx), name + "_grad_psi": np32(gpsi)})
    x = torch.zeros(1, 4)
    y = torch.zeros(96, 4)
    y[:, 0] = 100.0
    y[0, 0], y[64, 0] = 1.0, -1.0
    _, idx = c_transform_fwd(x, y, torch.zeros(96), autotune=False, block_n=32)
    out["tie_y"], out["tie_idx"] = np32(y), idx.numpy().astype(np.int64)
    save("c_transform_small", **out)


def gen_legacy():
    """OTT-convention legacy surface: the signed log-sum-exp kernels of kernels/sinkhorn_triton_ott_sqeuclid.py
    (interpreter run, manual blocks) next to the dense functions of testing/reference_sinkhorn.py:12-89 that the
    reference's test_sinkhorn_triton.py compares them with; the deprecated OTT-convention plan applications of
    kernels/apply_ott.py:213-450; the deprecated solver facade; and the trust-region CG of cg.py:201-369."""
    import warnings

    from flash_sinkhorn.cg import steihaug_cg
    from flash_sinkhorn.kernels.apply_ott import apply_plan_mat_sqeuclid, apply_plan_vec_sqeuclid
    from flash_sinkhorn.kernels.sinkhorn_triton_ott_sqeuclid import (
        apply_lse_kernel_sqeuclid,
        apply_transport_from_potentials_sqeuclid,
        sinkhorn_potentials_sqeuclid,
        update_potential,
    )

    warnings.simplefilter("ignore", DeprecationWarning)
    man = dict(block_m=32, block_n=32, block_k=16)
    n, m, d, eps = 37, 29, 8, 0.5
    gen = torch.Generator().manual_seed(91)
    x, y = torch.randn(n, d, generator=gen), 0.2 + torch.randn(m, d, generator=gen)
    f, g = torch.randn(n, generator=gen), torch.randn(m, generator=gen)
    vec_m, vec_n = torch.randn(m, generator=gen), torch.randn(n, generator=gen)
    vec_m[3], vec_n[5] = 0.0, 0.0
    out = dict(x=np32(x), y=np32(y), f=np32(f), g=np32(g), vec_m=np32(vec_m), vec_n=np32(vec_n), eps=np.float64(eps))
    for axis, vec in ((1, vec_m), (0, vec_n)):
        o, s = apply_lse_kernel_sqeuclid(x, y, f, g, eps, axis, **man)
        out[f"lse_axis{axis}"], out[f"lse_sgn_axis{axis}"] = np32(o), np32(s)
        o, s = apply_lse_kernel_sqeuclid(x, y, f, g, eps, axis, vec=vec, **man)
        out[f"vlse_axis{axis}"], out[f"vlse_sgn_axis{axis}"] = np32(o), np32(s)
        o, s = reference_sinkhorn.apply_lse_kernel_ref(x, y, f, g, eps, axis, vec=vec)
        out[f"vlse_dense_axis{axis}"], out[f"vlse_dense_sgn_axis{axis}"] = np32(o), np32(s)
    # all-positive and all-zero weight vectors: the sign is +1 everywhere, resp. 0 with -inf values
    o, s = apply_lse_kernel_sqeuclid(x, y, f, g, eps, 1, vec=torch.zeros(m), **man)
    out["zero_vec_lse"], out["zero_vec_sgn"] = np32(o), np32(s)

    loga = torch.log_softmax(torch.randn(n, generator=gen), 0)
    logb = torch.log_softmax(torch.randn(m, generator=gen), 0)
    out["loga"], out["logb"] = np32(loga), np32(logb)
    out["update_g"] = np32(update_potential(x, y, f, g, logb, eps, axis=0, **man))
    out["update_f"] = np32(update_potential(x, y, f, g, loga, eps, axis=1, **man))
    out["update_g_dense"] = np32(reference_sinkhorn.update_potential_ref(x, y, f, g, logb, eps, axis=0))

    fo, go = reference_sinkhorn.sinkhorn_potentials_ref(x, y, loga, logb, eps, n_iters=6)
    out["ott_f_dense"], out["ott_g_dense"] = np32(fo), np32(go)
    ff, gf = sinkhorn_potentials_sqeuclid(x, y, loga, logb, eps, 6, autotune=False)
    out["ott_f_facade"], out["ott_g_facade"] = np32(ff), np32(gf)
    out["transport_axis1"] = np32(apply_transport_from_potentials_sqeuclid(x, y, fo, go, vec_m, eps, 1, **man))
    out["transport_axis0"] = np32(apply_transport_from_potentials_sqeuclid(x, y, fo, go, vec_n, eps, 0, **man))
    out["transport_dense_axis1"] = np32(
        reference_sinkhorn.apply_transport_from_potentials_ref(x, y, fo, go, vec_m, eps, 1))

    cs = 0.5
    fh, gh = reference_sinkhorn.sinkhorn_potentials_ref(
        x * math.sqrt(cs), y * math.sqrt(cs), loga, logb, eps, n_iters=6)  # OTT potentials for cost cs*|x-y|^2
    mat_m, mat_n = torch.randn(m, d, generator=gen), torch.randn(n, d, generator=gen)
    scale = torch.rand(m, generator=gen) + 0.5
    out.update(cs=np.float64(cs), cs_f=np32(fh), cs_g=np32(gh), mat_m=np32(mat_m), mat_n=np32(mat_n),
               scale=np32(scale))
    out["dep_vec_axis1"] = np32(apply_plan_vec_sqeuclid(x, y, fh, gh, vec_m, eps=eps, axis=1, cost_scale=cs,
                                                        log_a=loga, log_b=logb))
    out["dep_vec_axis0"] = np32(apply_plan_vec_sqeuclid(x, y, fh, gh, vec_n, eps=eps, axis=0, cost_scale=cs))
    out["dep_mat_axis1"] = np32(apply_plan_mat_sqeuclid(x, y, fh, gh, mat_m, eps=eps, axis=1, cost_scale=cs,
                                                        scale=scale, log_a=loga, log_b=logb, autotune=False,
                                                        block_d=16, **man))
    out["dep_mat_axis0"] = np32(apply_plan_mat_sqeuclid(x, y, fh, gh, mat_n, eps=eps, axis=0, cost_scale=cs,
                                                        autotune=False, block_d=16, **man))
    save("legacy_ott_small", **out)

    # Trust-region CG on small dense symmetric matrices (float64), one case per way of stopping.
    cases = {}
    for name, (shift, delta, max_iter, rtol) in {
        "interior": (0.5, 50.0, 100, 1e-3), "boundary": (0.5, 0.3, 100, 1e-6), "negcurv": (-1.4, 1.0, 100, 1e-6),
        "maxiter": (0.5, 50.0, 2, 1e-6),
    }.items():
        gen = torch.Generator().manual_seed(17)
        B = torch.randn(30, 30, generator=gen, dtype=torch.float64)
        H = B @ B.T / 30 + shift * torch.eye(30, dtype=torch.float64)
        gr = torch.randn(30, generator=gen, dtype=torch.float64)
        p, info = steihaug_cg(lambda v: H @ v, gr, delta, max_iter=max_iter, rtol=rtol, atol=1e-12)
        print("steihaug", name, info)
        cases.update({f"{name}_H": H.numpy(), f"{name}_g": gr.numpy(), f"{name}_p": p.numpy(),
                      f"{name}_args": np.array([delta, max_iter, rtol], np.float64),
                      f"{name}_reason": np.array(info.termination_reason),
                      f"{name}_info": np.array([info.converged, info.iters, info.residual, info.hit_boundary,
                                                info.negative_curvature_detected, info.predicted_reduction],
                                               np.float64)})
    save("steihaug_small", **cases)


def gen_signatures():
    """Parameter names, kinds and defaults of every public callable of the reference's import surface, as
    JSON (tests/test_import_surface.py compares the package's own signatures with it)."""
    import importlib
    import inspect
    import json
    import warnings

    surface = {
        "samples_loss": ["SamplesLoss"],
        "cg": ["conjugate_gradient", "steihaug_cg"],
        "hvp": ["geomloss_to_ott_potentials", "hvp_x_sqeuclid", "hvp_x_sqeuclid_from_potentials",
                "inverse_hvp_x_sqeuclid_from_potentials"],
        "implicit_grad": ["implicit_grad_x", "implicit_grad_x_from_potentials"],
        "c_transform": ["c_transform_fwd", "c_transform_cost"],
        "sinkhorn_solvers": ["sinkhorn_flashstyle_alternating", "sinkhorn_flashstyle_symmetric"],
        "kernels._common": ["dampening", "log_weights", "max_diameter", "epsilon_schedule"],
        "kernels.sinkhorn_flashstyle_sqeuclid": [
            "flashsinkhorn_lse", "flashsinkhorn_lse_fused", "flashsinkhorn_symmetric_step",
            "precompute_flashsinkhorn_inputs", "compute_bias_f", "compute_bias_g",
            "shifted_to_standard_potentials", "standard_to_shifted_potentials"],
        "kernels.apply_flash": ["apply_plan_vec_flashstyle", "apply_plan_mat_flashstyle"],
        "kernels.apply_ott": ["mat5_sqeuclid", "apply_plan_vec_sqeuclid", "apply_plan_mat_sqeuclid"],
        "kernels.sinkhorn_triton_grad_sqeuclid": ["sinkhorn_geomloss_online_grad_sqeuclid"],
        "kernels.c_transform_sqeuclid": ["c_transform_kernel"],
        "kernels.sinkhorn_triton_ott_sqeuclid": ["sinkhorn_potentials_sqeuclid", "apply_lse_kernel_sqeuclid",
                                                 "update_potential", "apply_transport_from_potentials_sqeuclid"],
        "kernels.sinkhorn_triton_geomloss_sqeuclid": ["sinkhorn_geomloss_online_potentials_sqeuclid",
                                                      "geomloss_to_ott_potentials", "ott_to_geomloss_potentials"],
    }
    table = {}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for module, names in surface.items():
            mod = importlib.import_module("flash_sinkhorn." + module)
            for name in names:
                obj = getattr(mod, name)
                fn = obj.__init__ if inspect.isclass(obj) else obj
                table[f"{module}:{name}"] = [
                    [p.name, p.kind.name, None if p.default is inspect.Parameter.empty else repr(p.default)]
                    for p in inspect.signature(fn).parameters.values() if p.name != "self"]
    path = os.path.join(HERE, "api_signatures.json")
    with open(path, "w") as fh:
        json.dump(table, fh, sort_keys=True, separators=(",", ":"))
    print(f"wrote {path} ({os.path.getsize(path)} bytes, {len(table)} callables)")


HOST_CTOR_CASES = [
    dict(),
    dict(blur=0.1, reach=2.0, reach_x=0.5, half_cost=True),
    dict(blur=0.2, reach=1.5),
    dict(reach_x=1.0),
    dict(reach_y=3.0, debias=True),
    dict(backend="alternating", use_epsilon_scaling=False, eps=0.1, n_iters=7),
    dict(backend="alternating"),
    dict(backend="alternating", use_epsilon_scaling=False),
    dict(backend="triton"),
    dict(backend="auto", use_flashstyle=False),
    dict(backend="keops"),
    dict(loss="gaussian"),
    dict(p=1),
    dict(reach=-1.0),
    dict(reach_x=0.0),
    dict(reach_y=-2.0),
    dict(use_epsilon_scaling=False, eps=0.25, n_iters=9, potentials=True, normalize=False),
    dict(eps_list=[1.0, 0.5, 0.25], n_iters=2),
    dict(diameter=3.0, blur=0.3, scaling=0.7, threshold=1e-3, inner_iterations=4),
    dict(last_extrapolation=False, allow_tf32=False, hvp_max_cg_iter=20, hvp_tau2=1e-4),
    dict(lambda_x=0.7, lambda_y=1.8),
    dict(backend="alternating", use_epsilon_scaling=False, eps=0.1, n_iters=7, label_cost_matrix="eye3"),
]

HOST_ARG_CASES = [
    ("xy", dict(normalize=True)),
    ("axby", dict(normalize=True)),
    ("axby", dict(normalize=False)),
    ("axby_col", dict(normalize=True)),
    ("batched_xy", dict(normalize=True)),
    ("batched_axby", dict(normalize=True)),
    ("batched_axby_col", dict(normalize=False)),
    ("three_args", dict(normalize=True)),
    ("int_x", dict(normalize=True)),
    ("not_tensor", dict(normalize=True)),
    ("bad_ndim", dict(normalize=True)),
    ("batched_x_flat_y", dict(normalize=True)),
    ("batch_mismatch", dict(normalize=True)),
    ("dim_mismatch", dict(normalize=True)),
    ("bad_a", dict(normalize=True)),
    ("bad_b_batched", dict(normalize=True)),
]


def host_arg_case(name):
    """Inputs of one ``_process_args`` case; tests/test_host_api.py rebuilds them with the same seeded draws."""
    g = torch.Generator().manual_seed(5)
    x, y = torch.randn(6, 3, generator=g), torch.randn(4, 3, generator=g)
    a, b = torch.rand(6, generator=g) + 0.1, torch.rand(4, generator=g) + 0.1
    xb, yb = torch.randn(2, 6, 3, generator=g), torch.randn(2, 4, 3, generator=g)
    ab, bb = torch.rand(2, 6, generator=g) + 0.1, torch.rand(2, 4, generator=g) + 0.1
    return {
        "xy": (x, y), "axby": (a, x, b, y), "axby_col": (a[:, None], x, b[:, None], y),
        "batched_xy": (xb, yb), "batched_axby": (ab, xb, bb, yb),
        "batched_axby_col": (ab[..., None], xb, bb[..., None], yb),
        "three_args": (a, x, y), "int_x": (x.long(), y), "not_tensor": (x.tolist(), y),
        "bad_ndim": (x[0], y[0]), "batched_x_flat_y": (xb, y), "batch_mismatch": (xb, yb[:1]),
        "dim_mismatch": (x, y[:, :2]), "bad_a": (a[:5], x, b, y), "bad_b_batched": (ab, xb, bb[:, :3], yb),
    }[name]


def gen_host_api():
    """Host logic of SamplesLoss that needs no device: what the constructor accepts, warns about and derives
    (samples_loss.py:260-414), how ``_process_args`` parses and normalises the call forms (:73-191), and the
    schedule ``_eps_list_for_inputs`` builds (:451-470). Outcomes are stored as JSON."""
    import json
    import warnings

    from flash_sinkhorn.samples_loss import _process_args

    def plain(v):
        if torch.is_tensor(v):
            return {"tensor": list(v.shape)}
        return v

    ctor = []
    for kw in HOST_CTOR_CASES:
        real = {k: (torch.eye(3) if v == "eye3" else v) for k, v in kw.items()}
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter("always")
            try:
                obj = SamplesLoss(real.pop("loss", "sinkhorn"), **real)
                attrs = {k: plain(v) for k, v in vars(obj).items() if not k.startswith("_") and k != "training"}
                out = {"attrs": attrs}
            except Exception as e:  # noqa: BLE001 - the exception type IS the recorded outcome
                out = {"error": type(e).__name__}
        out["warnings"] = sorted({w.category.__name__ for w in caught})
        ctor.append({"kwargs": kw, **out})

    parsed = []
    for name, opt in HOST_ARG_CASES:
        try:
            p = _process_args(*host_arg_case(name), **opt)
            out = {"batched": bool(p.batched), "x_shape": list(p.x.shape), "y_shape": list(p.y.shape),
                   "a": p.a.double().tolist(), "b": p.b.double().tolist(),
                   "a_view_shape": list(p.a_view_shape), "b_view_shape": list(p.b_view_shape)}
        except Exception as e:  # noqa: BLE001
            out = {"error": type(e).__name__}
        parsed.append({"case": name, "options": opt, **out})

    g = torch.Generator().manual_seed(6)
    x, y = torch.randn(50, 4, generator=g), 0.5 + torch.randn(40, 4, generator=g)
    sched = []
    for kw in (dict(blur=0.3, scaling=0.6), dict(blur=0.3, scaling=0.6, n_iters=4), dict(diameter=3.0, blur=0.2),
               dict(use_epsilon_scaling=False, eps=0.25, n_iters=9), dict(eps_list=[1.0, 0.5, 0.25], n_iters=2),
               dict(use_epsilon_scaling=False), dict(blur=0.3, n_iters=0)):
        try:
            out = {"eps_list": [float(e) for e in SamplesLoss("sinkhorn", **kw)._eps_list_for_inputs(x, y)]}
        except Exception as e:  # noqa: BLE001
            out = {"error": type(e).__name__}
        sched.append({"kwargs": kw, **out})
    path = os.path.join(HERE, "host_api.json")
    with open(path, "w") as fh:
        json.dump({"constructor": ctor, "process_args": parsed, "schedule": sched,
                   "schedule_x": x.tolist(), "schedule_y": y.tolist()}, fh, sort_keys=True, separators=(",", ":"))
    print(f"wrote {path} ({os.path.getsize(path)} bytes)")
    for c in ctor:
        print("  ctor", c["kwargs"], c.get("error", "ok"), c["warnings"])
    for c in parsed:
        print("  args", c["case"], c.get("error", "ok"))
    for c in sched:
        print("  sched", c["kwargs"], c.get("error", len(c.get("eps_list", []))))


def gen_dense_reference():
    """The reference's dense oracles alone (no Triton): symmetric potentials, OTT alternating, gradients."""
    n, m, d = 128, 96, 32
    x, y, a, b = clouds(51, n, m, d, shift=0.1, weights="softmax")
    out = dict(x=np32(x), y=np32(y), a=np32(a), b=np32(b))
    f, g = reference_sinkhorn.sinkhorn_geomloss_potentials_ref(x, y, a, b, blur=0.4, scaling=0.6)
    out["sym_f"], out["sym_g"] = np32(f), np32(g)
    f, g = reference_sinkhorn.sinkhorn_geomloss_potentials_ref(x, y, a, b, use_epsilon_scaling=False, eps=0.3,
                                                               n_iters=20, last_extrapolation=False)
    out["fix_f"], out["fix_g"] = np32(f), np32(g)
    gx, gy = reference_sinkhorn.sinkhorn_geomloss_barycentric_grads_ref(x, y, a, b, f, g, eps=0.3)
    out["bary_gx"], out["bary_gy"] = np32(gx), np32(gy)
    fo, go = reference_sinkhorn.sinkhorn_potentials_ref(x, y, a.log(), b.log(), 0.3, 15)
    out["ott_f"], out["ott_g"] = np32(fo), np32(go)
    save("dense_reference", **out)


def gen_config1():
    """Benchmark configuration 1 (n=m=4096, d=64, eps=0.01, half cost, debias, 100 fixed iterations) with the
    reference's dense fp32 functions. Inputs are NOT stored: CPU generator seed 0, x then y."""
    t0 = time.time()
    gen = torch.Generator().manual_seed(0)
    n = m = 4096
    d = 64
    x = torch.randn(n, d, generator=gen)
    y = torch.randn(m, d, generator=gen)
    a = torch.full((n,), 1.0 / n)
    b = torch.full((m,), 1.0 / m)
    eps, iters = 0.01, 100
    s = math.sqrt(0.5)  # half cost == squared distance of inputs scaled by sqrt(1/2) (exact scaling of the cost)

    def solve(p, q, wp, wq):
        eps_list = [eps] * iters
        ps, qs = p * s, q * s
        f_pre, g_pre = reference_sinkhorn.sinkhorn_geomloss_potentials_ref(
            ps, qs, wp, wq, use_epsilon_scaling=False, eps=eps, n_iters=iters, last_extrapolation=False)
        f, g = reference_sinkhorn.sinkhorn_geomloss_potentials_ref(
            ps, qs, wp, wq, use_epsilon_scaling=False, eps=eps, n_iters=iters, last_extrapolation=True)
        cost = (wp * f).sum() + (wq * g).sum()
        gp, gq = reference_sinkhorn.sinkhorn_geomloss_barycentric_grads_ref(ps, qs, wp, wq, f_pre, g_pre, eps)
        return cost.item(), gp * s, gq * s  # chain rule through the sqrt(1/2) scaling

    c_xy, gx_xy, _ = solve(x, y, a, b)
    c_xx, gx_xx, gy_xx = solve(x, x, a, a)
    c_yy, _, _ = solve(y, y, b, b)
    loss = c_xy - 0.5 * c_xx - 0.5 * c_yy
    grad_x = gx_xy - 0.5 * (gx_xx + gy_xx)
    print(f"config1: OT_xy={c_xy!r} OT_xx={c_xx!r} OT_yy={c_yy!r} loss={loss!r} |grad|={grad_x.norm().item()!r} "
          f"({time.time() - t0:.0f}s)")
    save("config1", ot_xy=np.float64(c_xy), ot_xx=np.float64(c_xx), ot_yy=np.float64(c_yy), loss=np.float64(loss),
         grad_x_norm=np.float64(grad_x.norm().item()), grad_x_head=np32(grad_x[:16]),
         grad_x_rowsum=np32(grad_x.sum(dim=1)))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--skip-c1", action="store_true", help="skip the 4096x4096 dense solves (several minutes)")
    ap.add_argument("--only", default="", help="comma list of: kernels,solvers,loss,hvp,implicit,ctransform,labels,legacy,signatures,hostapi,dense,c1")
    args = ap.parse_args()
    which = set(args.only.split(",")) if args.only else {"kernels", "solvers", "loss", "hvp", "implicit",
                                                         "ctransform", "labels", "legacy", "signatures", "hostapi", "dense", "c1"}
    print("reference version", flash_sinkhorn.__version__, "from", os.path.dirname(flash_sinkhorn.__file__))
    if "dense" in which:
        gen_dense_reference()
    if "kernels" in which:
        gen_kernels()
    if "solvers" in which:
        gen_solvers()
    if "loss" in which:
        gen_samples_loss()
    if "hvp" in which:
        gen_hvp()
    if "implicit" in which:
        gen_implicit()
    if "ctransform" in which:
        gen_c_transform()
    if "labels" in which:
        gen_label_cost()
    if "legacy" in which:
        gen_legacy()
    if "signatures" in which:
        gen_signatures()
    if "hostapi" in which:
        gen_host_api()
    if "c1" in which and not args.skip_c1:
        gen_config1()
    sys.exit(0)
