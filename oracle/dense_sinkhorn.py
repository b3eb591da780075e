"""Dense CPU oracle for the streaming-Sinkhorn hot path.  TEST INFRASTRUCTURE ONLY.

A plain numpy (float64 by default) restatement of what the reference package
ot-triton-lab/flash-sinkhorn computes on this path, with the full n x m matrices
materialised. Nothing under ``flash_sinkhorn_b200`` may import it: it is the checker
for ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``, never a product code path.

Parity status: PINNED. ``tests/test_oracle_golden.py`` checks every function below
against fixtures under ``tests/golden/`` that were produced by importing the reference
itself (its dense PyTorch oracles, and its Triton kernels under the Triton CPU
interpreter) with ``tests/golden/make_golden.py``.

Each function cites the reference file:line it follows (paths relative to the
reference's ``src/flash_sinkhorn/``). Notation: cs = cost_scale,
C_ij = cs*|x_i-y_j|^2, alpha = cs*|x|^2, beta = cs*|y|^2, f_hat = f-alpha, g_hat = g-beta.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np

LOG_ZERO_WEIGHT = -100000.0


# --------------------------------------------------------------------------- host scalars
def dampening(eps: float, rho: Optional[float]) -> float:
    """kernels/_common.py:20-36."""
    return 1.0 if rho is None else 1.0 / (1.0 + eps / rho)


def log_weights(w: np.ndarray) -> np.ndarray:
    """kernels/_common.py:39-44 (non-positive weights -> -1e5, not -inf)."""
    w = np.asarray(w)
    out = np.full(w.shape, LOG_ZERO_WEIGHT, dtype=w.dtype)
    pos = w > 0
    out[pos] = np.log(w[pos])
    return out


def max_diameter(x: np.ndarray, y: np.ndarray) -> float:
    """kernels/_common.py:47-53: diagonal of the joint bounding box, evaluated in fp32."""
    x32, y32 = np.asarray(x, np.float32), np.asarray(y, np.float32)
    lo = np.minimum(x32.min(axis=0), y32.min(axis=0))
    hi = np.maximum(x32.max(axis=0), y32.max(axis=0))
    return float(np.sqrt(np.sum((hi - lo).astype(np.float32) ** 2, dtype=np.float32)))


def epsilon_schedule(diameter: float, blur: float, scaling: float, p: float = 2.0):
    """kernels/_common.py:56-90."""
    ladder = [float(np.exp(e)) for e in np.arange(p * np.log(diameter), p * np.log(blur), p * np.log(scaling))]
    return [diameter**p] + ladder + [blur**p]


# --------------------------------------------------------------------------- building blocks
def sqnorm(x: np.ndarray) -> np.ndarray:
    return np.sum(x * x, axis=1)


def _lse(vals: np.ndarray, axis: int) -> np.ndarray:
    mx = np.max(vals, axis=axis, keepdims=True)
    mx = np.where(np.isfinite(mx), mx, 0.0)
    return np.squeeze(mx, axis=axis) + np.log(np.sum(np.exp(vals - mx), axis=axis))


def lse_update(x, y, bias, eps, cost_scale=1.0, damping=1.0):
    """kernels/sinkhorn_flashstyle_sqeuclid.py:199-307 (K1):
    out_i = -eps*damping*LSE_j[(2cs/eps) x_i.y_j + bias_j]."""
    logits = (2.0 * cost_scale / eps) * (x @ y.T) + bias[None, :]
    return -eps * damping * _lse(logits, axis=1)


def lse_update_fused(x, y, g_hat, log_w, eps, cost_scale=1.0, damping=1.0):
    """kernels/sinkhorn_flashstyle_sqeuclid.py:322-419 (K2): bias_j = g_hat_j/eps + log_w_j."""
    return lse_update(x, y, g_hat / eps + log_w, eps, cost_scale, damping)


def symmetric_step(x, y, f_hat, g_hat, log_a, log_b, eps, cost_scale=1.0, alpha=0.5, damping_f=1.0,
                   damping_g=1.0):
    """kernels/sinkhorn_flashstyle_sqeuclid.py:438-661 (K3): both candidates from the OLD potentials,
    new = (1-alpha)*old + alpha*cand; no shift correction inside the kernel."""
    cf = lse_update_fused(x, y, g_hat, log_b, eps, cost_scale, damping_f)
    cg = lse_update_fused(y, x, f_hat, log_a, eps, cost_scale, damping_g)
    return (1.0 - alpha) * f_hat + alpha * cf, (1.0 - alpha) * g_hat + alpha * cg


# --------------------------------------------------------------------------- solvers
def solve_symmetric(x, y, a, b, eps_list: Sequence[float], *, last_extrapolation=True, cost_scale=1.0,
                    rho_x=None, rho_y=None, threshold=None, check_every=5, f_init=None, g_init=None) -> Dict:
    """sinkhorn_solvers.py:290-707. Step sequence :476-554: init step (weight 1) at eps_list[0];
    one weight-1/2 step per eps; final weight-1 step at eps_list[-1]. Unbalanced shift correction
    :509-517; early stop :521-531 (first check only stores the snapshot); prelast :533-536."""
    dt = x.dtype
    alpha, beta = cost_scale * sqnorm(x), cost_scale * sqnorm(y)
    log_a, log_b = log_weights(a).astype(dt), log_weights(b).astype(dt)
    f_hat = (-alpha if f_init is None else np.asarray(f_init, dt) - alpha).copy()
    g_hat = (-beta if g_init is None else np.asarray(g_init, dt) - beta).copy()

    def step(fh, gh, eps, w):
        df, dg = dampening(eps, rho_x), dampening(eps, rho_y)
        nf, ng = symmetric_step(x, y, fh, gh, log_a, log_b, eps, cost_scale, w, df, dg)
        if df < 1.0:
            nf = nf - w * alpha * (1.0 - df)
        if dg < 1.0:
            ng = ng - w * beta * (1.0 - dg)
        return nf.astype(dt), ng.astype(dt)

    used = 0
    f_hat, g_hat = step(f_hat, g_hat, eps_list[0], 1.0)
    used += 1
    prev = None
    for i, eps in enumerate(eps_list):
        f_hat, g_hat = step(f_hat, g_hat, eps, 0.5)
        used += 1
        if threshold is not None and (i + 1) % check_every == 0:
            if prev is None:
                prev = (f_hat.copy(), g_hat.copy())
            else:
                change = max(np.abs(f_hat - prev[0]).max(), np.abs(g_hat - prev[1]).max())
                if change < threshold:
                    break
                prev = (f_hat.copy(), g_hat.copy())
    out = {}
    if last_extrapolation:
        out["f_pre"], out["g_pre"] = f_hat + alpha, g_hat + beta
        f_hat, g_hat = step(f_hat, g_hat, eps_list[-1], 1.0)
        used += 1
    out.update(f=f_hat + alpha, g=g_hat + beta, n_iters=used)
    if not last_extrapolation:
        out["f_pre"], out["g_pre"] = out["f"], out["g"]
    return out


def expand_tile_mask(tile_mask: np.ndarray, n: int, m: int, tile: int = 128) -> np.ndarray:
    """Boolean [ceil(n/tile), ceil(m/tile)] -> boolean [n, m] (True = entry kept)."""
    return np.kron(tile_mask.astype(bool), np.ones((tile, tile), dtype=bool))[:n, :m]


def solve_alternating(x, y, a, b, eps_list: Sequence[float], iters_per_eps: int, *, cost_scale=1.0, rho_x=None,
                      rho_y=None, ott_convention=False, threshold=None, check_every=5, tile_mask=None) -> Dict:
    """sinkhorn_solvers.py:30-287 for one eps (GeomLoss convention :240-259, OTT convention :188-228;
    damped updates get NO shift correction). Several eps = the same loop warm-started per eps
    (annealed alternating and tile masks have no reference implementation: composition of the
    reference's primitives, dropped tiles contribute exp(-inf) = 0)."""
    dt = x.dtype
    n, m = x.shape[0], y.shape[0]
    alpha, beta = cost_scale * sqnorm(x), cost_scale * sqnorm(y)
    log_a, log_b = log_weights(a).astype(dt), log_weights(b).astype(dt)
    f_hat, g_hat = -alpha.copy(), -beta.copy()
    xy = x @ y.T
    if tile_mask is not None:
        keep = expand_tile_mask(tile_mask, n, m)
        neg = np.where(keep, 0.0, -np.inf)
    else:
        neg = 0.0
    prev = (f_hat.copy(), g_hat.copy())
    used, it_global, stop = 0, 0, False
    for eps in eps_list:
        df, dg = dampening(eps, rho_x), dampening(eps, rho_y)
        sc = 2.0 * cost_scale / eps
        for _ in range(iters_per_eps):
            if ott_convention:
                g_hat = eps * log_b - eps * dg * _lse(sc * xy + (f_hat / eps)[:, None] + neg, axis=0)
                f_hat = eps * log_a - eps * df * _lse(sc * xy + (g_hat / eps)[None, :] + neg, axis=1)
            else:
                f_hat = -eps * df * _lse(sc * xy + (g_hat / eps + log_b)[None, :] + neg, axis=1)
                g_hat = -eps * dg * _lse(sc * xy + (f_hat / eps + log_a)[:, None] + neg, axis=0)
            f_hat, g_hat = f_hat.astype(dt), g_hat.astype(dt)
            used += 1
            it_global += 1
            if threshold is not None and it_global % check_every == 0:
                change = max(np.abs(f_hat - prev[0]).max(), np.abs(g_hat - prev[1]).max())
                if change < threshold:
                    stop = True
                    break
                prev = (f_hat.copy(), g_hat.copy())
        if stop:
            break
    return dict(f=f_hat + alpha, g=g_hat + beta, n_iters=used)


# --------------------------------------------------------------------------- cost
def ot_cost(a, b, f, g, eps, rho_x=None, rho_y=None) -> float:
    """_autograd.py:436-455: <a,f>+<b,g> when at most one side is relaxed, else
    (rho+eps/2)*<w, 1-exp(-pot/rho)> per side."""
    if rho_x is None or rho_y is None:
        return float(np.sum(a * f) + np.sum(b * g))
    return float((rho_x + eps / 2) * np.sum(a * (1 - np.exp(-f / rho_x)))
                 + (rho_y + eps / 2) * np.sum(b * (1 - np.exp(-g / rho_y))))


def samples_loss(x, y, a, b, eps_list, *, cost_scale=1.0, rho_x=None, rho_y=None, debias=False,
                 last_extrapolation=True, threshold=None, check_every=10, want_grad_x=False) -> Dict:
    """samples_loss.py:494-512 (debias = OT(x,y) - OT(x,x)/2 - OT(y,y)/2) over _autograd.py:307-455;
    gradient as in _autograd.py:458-506 (prelast potentials; the self term contributes gx+gy)."""
    eps = float(eps_list[-1])

    def one(p, q, wp, wq):
        s = solve_symmetric(p, q, wp, wq, eps_list, last_extrapolation=last_extrapolation, cost_scale=cost_scale,
                            rho_x=rho_x, rho_y=rho_y, threshold=threshold, check_every=check_every)
        return ot_cost(wp, wq, s["f"], s["g"], eps, rho_x, rho_y), s

    c_xy, s_xy = one(x, y, a, b)
    out = dict(loss=c_xy, ot_xy=c_xy)
    if want_grad_x:
        gx, _ = grad_xy(x, y, a, b, s_xy["f_pre"], s_xy["g_pre"], eps, cost_scale)
        out["grad_x"] = gx
    if debias:
        c_xx, s_xx = one(x, x, a, a)
        c_yy, _ = one(y, y, b, b)
        out.update(loss=c_xy - 0.5 * c_xx - 0.5 * c_yy, ot_xx=c_xx, ot_yy=c_yy)
        if want_grad_x:
            g1, g2 = grad_xy(x, x, a, a, s_xx["f_pre"], s_xx["g_pre"], eps, cost_scale)
            out["grad_x"] = out["grad_x"] - 0.5 * (g1 + g2)
    return out


# --------------------------------------------------------------------------- gradient
def grad_xy(x, y, a, b, f, g, eps, cost_scale=1.0, grad_scale=1.0):
    """kernels/sinkhorn_triton_grad_sqeuclid.py:102-402 (same formula as
    testing/reference_sinkhorn.py:208-233 times cs): softmax-normalised barycentres,
    grad_x_i = 2cs*gs*a_i*(x_i - ybar_i); non-positive weights use log = -1e5."""
    C = cost_scale * (sqnorm(x)[:, None] + sqnorm(y)[None, :] - 2.0 * (x @ y.T))
    lw_xy = (g[None, :] - C) / eps + log_weights(b)[None, :]
    w = np.exp(lw_xy - lw_xy.max(axis=1, keepdims=True))
    ybar = (w @ y) / np.maximum(w.sum(axis=1, keepdims=True), 1e-40)
    gx = (2.0 * cost_scale * grad_scale) * a[:, None] * (x - ybar)
    lw_yx = (f[:, None] - C) / eps + log_weights(a)[:, None]
    w = np.exp(lw_yx - lw_yx.max(axis=0, keepdims=True))
    xbar = (w.T @ x) / np.maximum(w.sum(axis=0)[:, None], 1e-40)
    gy = (2.0 * cost_scale * grad_scale) * b[:, None] * (y - xbar)
    return gx, gy


# --------------------------------------------------------------------------- plan applications
def plan_shifted(x, y, f_hat, g_hat, log_a, log_b, eps, cost_scale=1.0):
    """kernels/apply_flash.py:86-99: P_ij = a_i b_j exp((f_hat_i + g_hat_j + 2cs x_i.y_j)/eps)."""
    return np.exp((f_hat[:, None] + g_hat[None, :] + 2.0 * cost_scale * (x @ y.T)) / eps
                  + log_a[:, None] + log_b[None, :])


def apply_vec(x, y, f_hat, g_hat, log_a, log_b, vec, eps, axis, cost_scale=1.0):
    """kernels/apply_flash.py:835-951."""
    P = plan_shifted(x, y, f_hat, g_hat, log_a, log_b, eps, cost_scale)
    return P @ vec if axis == 1 else P.T @ vec


def apply_mat(x, y, f_hat, g_hat, log_a, log_b, mat, eps, axis, cost_scale=1.0, scale=None):
    """kernels/apply_flash.py:360-579 (scale multiplies the rows of mat, axis 1 only)."""
    P = plan_shifted(x, y, f_hat, g_hat, log_a, log_b, eps, cost_scale)
    if axis == 1:
        return P @ (mat if scale is None else mat * scale[:, None])
    return P.T @ mat


def plan_ott(x, y, f, g, eps, cost_scale=1.0):
    """testing/reference_hvp.py:19-30: P = exp((f+g-C)/eps), weights inside f, g."""
    C = cost_scale * (sqnorm(x)[:, None] + sqnorm(y)[None, :] - 2.0 * (x @ y.T))
    return np.exp((f[:, None] + g[None, :] - C) / eps)


def signed_lse_ott(x, y, f, g, eps, axis, vec=None):
    """testing/reference_sinkhorn.py:12-62 and kernels/sinkhorn_triton_ott_sqeuclid.py:157-286, :482-690:
    eps*log|sum exp((f_i+g_j-C_ij)/eps)*vec| minus the potential of the kept index (non-finite ones count as 0),
    and the sign of the sum (all ones without vec; a zero sum gives -inf, sign 0). Cost is |x-y|^2."""
    C = sqnorm(x)[:, None] + sqnorm(y)[None, :] - 2.0 * (x @ y.T)
    logits = (f[:, None] + g[None, :] - C) / eps
    own = f if axis == 1 else g
    own = np.where(np.isfinite(own), own, 0.0)
    if vec is None:
        lse = _lse(logits, axis=axis)
        return eps * lse - own, np.ones_like(lse)
    with np.errstate(divide="ignore"):
        logv = np.where(vec != 0, np.log(np.abs(vec)), -np.inf)
    vals = logits + (logv[None, :] if axis == 1 else logv[:, None])
    sg = np.sign(vec)
    top = vals.max(axis=axis, keepdims=True)
    with np.errstate(invalid="ignore", divide="ignore"):
        # an all-zero vec makes every term exp(-inf - (-inf)) = NaN; the comparisons below are then all
        # False, which is how the reference ends up with (-inf, 0) for such rows
        s = np.sum((sg[None, :] if axis == 1 else sg[:, None]) * np.exp(vals - top), axis=axis)
        lse = np.where(np.abs(s) > 0, np.squeeze(top, axis=axis) + np.log(np.abs(s)), -np.inf)
    return eps * lse - own, np.where(s > 0, 1.0, np.where(s < 0, -1.0, 0.0))


def update_potential_ott(x, y, f, g, log_marginal, eps, axis):
    """testing/reference_sinkhorn.py:65-68, kernels/sinkhorn_triton_ott_sqeuclid.py:693-709."""
    lse, _ = signed_lse_ott(x, y, f, g, eps, axis)
    return eps * log_marginal - np.where(np.isfinite(lse), lse, 0.0)


def sinkhorn_potentials_ott(x, y, loga, logb, eps, n_iters):
    """testing/reference_sinkhorn.py:71-82: zero start, g-update then f-update, log-marginals absorbed."""
    f, g = np.zeros(x.shape[0], x.dtype), np.zeros(y.shape[0], y.dtype)
    for _ in range(n_iters):
        g = update_potential_ott(x, y, f, g, logb, eps, axis=0)
        f = update_potential_ott(x, y, f, g, loga, eps, axis=1)
    return f, g


def apply_transport_ott(x, y, f, g, vec, eps, axis):
    """testing/reference_sinkhorn.py:85-89, kernels/sinkhorn_triton_ott_sqeuclid.py:712-735: P vec or P^T vec."""
    lse, sg = signed_lse_ott(x, y, f, g, eps, axis, vec=vec)
    return sg * np.exp((lse + (f if axis == 1 else g)) / eps)


def mat5(x, y, f_ott, g_ott, A, eps, cost_scale=1.0):
    """kernels/apply_ott.py:35-168: (-4cs/eps) sum_j P_ij (A_i.y_j) y_j."""
    P = plan_ott(x, y, f_ott, g_ott, eps, cost_scale)
    return (-4.0 * cost_scale / eps) * ((P * (A @ y.T)) @ y)


# --------------------------------------------------------------------------- HVP
def conjugate_gradient(matvec, b, max_iter=300, rtol=1e-6, atol=1e-6):
    """cg.py:27-121 (x0 = 0, no preconditioner). Returns (x, converged, iters, res, res0)."""
    xk = np.zeros_like(b)
    r = b.copy()
    p = r.copy()
    rz = float(r @ r)
    r0 = float(np.linalg.norm(r))
    tol = max(atol, rtol * r0)
    for it in range(int(max_iter)):
        Ap = matvec(p)
        den = float(p @ Ap)
        if den == 0:
            break
        al = rz / den
        xk = xk + al * p
        r = r - al * Ap
        res = float(np.linalg.norm(r))
        if res <= tol:
            return xk, True, it + 1, res, r0
        rz_new = float(r @ r)
        p = r + (rz_new / rz) * p
        rz = rz_new
    return xk, False, int(max_iter), float(np.linalg.norm(r)), r0


def hvp_x(x, y, f_ott, g_ott, A, eps, *, rho_x=None, rho_y=None, cost_scale=1.0, tau2=1e-5, max_cg_iter=300,
          cg_rtol=1e-6, cg_atol=1e-6, direct_solve=False) -> Dict:
    """hvp.py:282-623 with the plan materialised (cf. testing/reference_hvp.py:155-356, which
    hard-codes cs = 1). direct_solve=True replaces CG by a dense linear solve."""
    e, c = float(eps), 2.0 * cost_scale
    P = plan_ott(x, y, f_ott, g_ott, e, cost_scale)
    a_hat, b_hat = P.sum(axis=1), P.sum(axis=0)
    kx = 1.0 if rho_x is None else (rho_x + e) / rho_x
    ky = 1.0 if rho_y is None else (rho_y + e) / rho_y
    floor = max(1e-12, e * 1e-10)
    Dx, Dy = kx * np.maximum(a_hat, floor), ky * np.maximum(b_hat, floor)
    denom = Dy + e * tau2 if (rho_x is None and rho_y is None) else Dy
    xa = np.sum(x * A, axis=1)
    Py = P @ y
    PtA = P.T @ A
    rx = c * (a_hat * xa - np.sum(A * Py, axis=1))
    ry = c * (P.T @ xa - np.sum(y * PtA, axis=1))
    y1 = rx / Dx
    rhs = ry - P.T @ y1

    def schur(z):
        return denom * z - P.T @ ((P @ z) / Dx)

    if direct_solve:
        S = np.diag(denom) - P.T @ (P / Dx[:, None])
        z = np.linalg.solve(S, rhs)
        conv, iters, res, r0 = True, 0, float(np.linalg.norm(schur(z) - rhs)), float(np.linalg.norm(rhs))
    else:
        z, conv, iters, res, r0 = conjugate_gradient(schur, rhs, max_cg_iter, cg_rtol, cg_atol)
    Pz = P @ z
    z1 = y1 - Pz / Dx
    Pyz = P @ (y * z[:, None])
    RTz = c * (x * (a_hat * z1)[:, None] - Py * z1[:, None] + x * Pz[:, None] - Pyz)
    k2 = 2.0 * c / e
    t1 = c * a_hat[:, None] * A
    t2 = -k2 * x * (xa * a_hat)[:, None]
    t3 = k2 * Py * xa[:, None]
    t4 = k2 * x * np.sum(Py * A, axis=1)[:, None]
    t5 = mat5(x, y, f_ott, g_ott, A, e, cost_scale)
    return dict(hvp=RTz / e + t1 + t2 + t3 + t4 + t5, cg_converged=conv, cg_iters=iters, cg_residual=res,
                cg_initial_residual=r0)


def inverse_hvp_x(x, y, f_ott, g_ott, gr, eps, *, cost_scale=1.0, tau2=1e-5, max_outer_iter=100,
                  outer_rtol=1e-6, outer_atol=1e-6, direct_solve=False) -> Dict:
    """hvp.py:696-835: outer CG on H z = gr with the HVP as operator (inner Schur systems solved densely).
    direct_solve=True assembles H column by column and solves the n*d x n*d system instead."""
    n, d = x.shape

    def hessian_times(flat):
        return hvp_x(x, y, f_ott, g_ott, flat.reshape(n, d), eps, cost_scale=cost_scale, tau2=tau2,
                     direct_solve=True)["hvp"].reshape(-1)

    b = gr.reshape(-1).astype(np.float64)
    if direct_solve:
        H = np.stack([hessian_times(col) for col in np.eye(n * d)], axis=1)
        z = np.linalg.solve(H, b)
        conv, iters, res, r0 = True, 0, float(np.linalg.norm(H @ z - b)), float(np.linalg.norm(b))
    else:
        z, conv, iters, res, r0 = conjugate_gradient(hessian_times, b, max_outer_iter, outer_rtol, outer_atol)
    return dict(z=z.reshape(n, d), cg_converged=conv, cg_iters=iters, cg_residual=res, cg_initial_residual=r0)


# --------------------------------------------------------------------------- OTDD label-augmented cost
def label_solve_symmetric(x, y, a, b, eps_list: Sequence[float], label_x, label_y, W, *, lambda_x=1.0,
                          lambda_y=1.0, cost_scale=1.0, last_extrapolation=True) -> Dict:
    """Balanced symmetric solve with the label term of kernels/sinkhorn_flashstyle_sqeuclid.py:545-560:
    logit_ij = (lambda_x*2cs*x_i.y_j - lambda_y*cs*W[lx_i, ly_j] + g_hat_j)/eps + log b_j, the shifts
    alpha = cs|x|^2, beta = cs|y|^2 NOT scaled by lambda_x (sinkhorn_solvers.py:463-470); same step
    sequence as solve_symmetric."""
    dt = x.dtype
    alpha, beta = cost_scale * sqnorm(x), cost_scale * sqnorm(y)
    log_a, log_b = log_weights(a).astype(dt), log_weights(b).astype(dt)
    core = lambda_x * 2.0 * cost_scale * (x @ y.T) - lambda_y * cost_scale * W[np.ix_(label_x, label_y)]
    f_hat, g_hat = -alpha.copy(), -beta.copy()

    def step(fh, gh, eps, w):
        cf = -eps * _lse((core + gh[None, :]) / eps + log_b[None, :], axis=1)
        cg = -eps * _lse((core + fh[:, None]) / eps + log_a[:, None], axis=0)
        return ((1 - w) * fh + w * cf).astype(dt), ((1 - w) * gh + w * cg).astype(dt)

    f_hat, g_hat = step(f_hat, g_hat, eps_list[0], 1.0)
    for eps in eps_list:
        f_hat, g_hat = step(f_hat, g_hat, eps, 0.5)
    out = dict(f_pre=f_hat + alpha, g_pre=g_hat + beta)
    if last_extrapolation:
        f_hat, g_hat = step(f_hat, g_hat, eps_list[-1], 1.0)
    out.update(f=f_hat + alpha, g=g_hat + beta)
    return out


def label_grad_xy(x, y, a, b, f, g, eps, label_x, label_y, W, *, lambda_x=1.0, lambda_y=1.0, cost_scale=1.0,
                  grad_scale=1.0):
    """kernels/sinkhorn_triton_grad_sqeuclid.py:225-236, :275: weights from the cost
    lambda_x*cs|x-y|^2 + lambda_y*cs*W[lx, ly]; grad_x_i = 2*lambda_x*cs*gs*a_i*(x_i - ybar_i)."""
    C = (lambda_x * cost_scale * (sqnorm(x)[:, None] + sqnorm(y)[None, :] - 2.0 * (x @ y.T))
         + lambda_y * cost_scale * W[np.ix_(label_x, label_y)])
    lw = (g[None, :] - C) / eps + log_weights(b)[None, :]
    w = np.exp(lw - lw.max(axis=1, keepdims=True))
    gx = (2.0 * lambda_x * cost_scale * grad_scale) * a[:, None] * (x - (w @ y) / w.sum(axis=1, keepdims=True))
    lw = (f[:, None] - C) / eps + log_weights(a)[:, None]
    w = np.exp(lw - lw.max(axis=0, keepdims=True))
    gy = (2.0 * lambda_x * cost_scale * grad_scale) * b[:, None] * (y - (w.T @ x) / w.sum(axis=0)[:, None])
    return gx, gy


def label_samples_loss(x, y, a, b, eps_list, label_x, label_y, W, *, lambda_x=1.0, lambda_y=1.0, cost_scale=1.0,
                       debias=False) -> Dict:
    """samples_loss.py:494-512 with labels: OT(x,y) uses (label_x, label_y), OT(x,x) (label_x, label_x),
    OT(y,y) (label_y, label_y); cost <a,f>+<b,g>; gradient from the pre-extrapolation potentials."""
    eps = float(eps_list[-1])
    kw = dict(lambda_x=lambda_x, lambda_y=lambda_y, cost_scale=cost_scale)

    def one(p, q, wp, wq, lp, lq):
        s = label_solve_symmetric(p, q, wp, wq, eps_list, lp, lq, W, **kw)
        return float(np.sum(wp * s["f"]) + np.sum(wq * s["g"])), s

    c_xy, s_xy = one(x, y, a, b, label_x, label_y)
    gx, _ = label_grad_xy(x, y, a, b, s_xy["f_pre"], s_xy["g_pre"], eps, label_x, label_y, W, **kw)
    out = dict(loss=c_xy, grad_x=gx)
    if debias:
        c_xx, s_xx = one(x, x, a, a, label_x, label_x)
        c_yy, _ = one(y, y, b, b, label_y, label_y)
        g1, g2 = label_grad_xy(x, x, a, a, s_xx["f_pre"], s_xx["g_pre"], eps, label_x, label_x, W, **kw)
        out.update(loss=c_xy - 0.5 * c_xx - 0.5 * c_yy, grad_x=gx - 0.5 * (g1 + g2))
    return out


# --------------------------------------------------------------------------- hard c-transform
def c_transform(x, y, psi, cost_scale=1.0):
    """c_transform.py:32-112 / kernels/c_transform_sqeuclid.py:117-206: c_i = min_j [cs|x_i-y_j|^2 - psi_j]
    evaluated in the factored form alpha_i + min_j(-2cs x_i.y_j + cs|y_j|^2 - psi_j); first minimiser."""
    inner = -2.0 * cost_scale * (x @ y.T) + (cost_scale * sqnorm(y) - psi)[None, :]
    idx = np.argmin(inner, axis=1)
    return cost_scale * sqnorm(x) + inner[np.arange(x.shape[0]), idx], idx.astype(np.int64)


def c_transform_cost(x, y, psi, a, b, cost_scale=1.0) -> Dict:
    """c_transform.py:115-174: L = <a, c^psi(x)> + <b, psi>; Danskin gradients at the arg-min."""
    c, idx = c_transform(x, y, psi, cost_scale)
    grad_x = (a * 2.0 * cost_scale)[:, None] * (x - y[idx])
    mass = np.zeros(y.shape[0])
    np.add.at(mass, idx, a)
    return dict(loss=float(a @ c + b @ psi), grad_x=grad_x, grad_psi=b - mass, c=c, idx=idx)


# --------------------------------------------------------------------------- implicit differentiation
def implicit_grad_x(x, y, f_hat, g_hat, grad_f, grad_g, log_a, log_b, eps, *, cost_scale=1.0, tau2=1e-5,
                    max_cg_iter=100, cg_rtol=1e-6, cg_atol=1e-6, direct_solve=False) -> Dict:
    """implicit_grad.py:36-242 with the plan materialised: marginals r, c; Schur system
    [diag(c + eps*tau2)/eps - P^T diag(1/r) P / eps] lam_g = grad_g - P^T (grad_f / r) (:176-194);
    lam_f = eps grad_f / r - P lam_g / r (:202);
    grad_x = (2/eps) [lam_f (x r - P y) + (P lam_g) x - P (lam_g y)] (:221-236)."""
    e = float(eps)
    P = plan_shifted(x, y, f_hat, g_hat, log_a, log_b, e, cost_scale)
    r, c = P.sum(axis=1), P.sum(axis=0)
    rhs = grad_g - P.T @ (grad_f / r)
    diag = (c + e * tau2) / e

    def schur(z):
        return diag * z - P.T @ ((P @ z) / r) / e

    if direct_solve:
        S = np.diag(diag) - P.T @ (P / r[:, None]) / e
        lam_g = np.linalg.solve(S, rhs)
        conv, iters, res = True, 0, float(np.linalg.norm(schur(lam_g) - rhs))
    else:
        lam_g, conv, iters, res, _ = conjugate_gradient(schur, rhs, max_cg_iter, cg_rtol, cg_atol)
    P_lam = P @ lam_g
    lam_f = e * grad_f / r - P_lam / r
    Py = P @ y
    Py_lam = P @ (y * lam_g[:, None])
    grad_x = (2.0 / e) * (lam_f[:, None] * (x * r[:, None] - Py) + P_lam[:, None] * x - Py_lam)
    return dict(grad_x=grad_x, cg_converged=conv, cg_iters=iters, cg_residual=res)
