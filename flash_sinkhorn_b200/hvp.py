"""Hessian-vector product of the entropic OT cost w.r.t. the source points.

Public surface of the reference's ``hvp.py``: ``HvpInfo`` (:44-52),
``geomloss_to_ott_potentials`` (:55-76), ``hvp_x_sqeuclid_from_potentials`` (:164-623),
``hvp_x_sqeuclid`` (:626-693). The algebra is the Schur-complement form the reference
uses (marginals, ``P y``, ``P^T A``, a CG solve on ``diag(denom) - P^T diag(1/D_x) P``,
back-substitution, then the five explicit terms); every plan application streams
through the CUDA engine and nothing of size n*m is formed.

With the default ``preconditioner="none"`` and no warm start the CG loop runs entirely
on the device (``fs_schur_cg``): dot products, the stopping test and the iteration
counter never visit the host, and the only synchronisation is reading the four-float
result record. Other preconditioners / ``cg_x0`` / ``cg_stabilise_every`` use the
host-driven ``conjugate_gradient``. The reference's optional dense / batched / compiled /
fused-matvec CG variants are accepted as keywords and ignored.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

from flash_sinkhorn_b200 import _lib
from flash_sinkhorn_b200.cg import CGInfo, conjugate_gradient
from flash_sinkhorn_b200.kernels._common import log_weights
from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
from flash_sinkhorn_b200.kernels.apply_ott import mat5_sqeuclid
from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric

__all__ = [
    "HvpInfo",
    "geomloss_to_ott_potentials",
    "ott_to_geomloss_potentials",
    "hvp_x_sqeuclid",
    "inverse_hvp_x_sqeuclid_from_potentials",
    "hvp_x_sqeuclid_from_potentials",
    "sinkhorn_prelast_potentials_sqeuclid",
]


@dataclass(frozen=True)
class HvpInfo:
    cg_converged: bool
    cg_iters: int
    cg_residual: float
    cg_initial_residual: float
    converged_lambda: float = 0.0
    hit_neg_curv: bool = False
    diagnostic_msg: str = ""


def geomloss_to_ott_potentials(f, g, a, b, *, eps: float):
    """``(f + eps*log a, g + eps*log b)``: absorb the weights so that ``P = exp((f+g-C)/eps)``."""
    e = float(eps)
    return f.float() + e * log_weights(a), g.float() + e * log_weights(b)


def ott_to_geomloss_potentials(f_hat, g_hat, a, b, *, eps: float):
    """Inverse of :func:`geomloss_to_ott_potentials`."""
    e = float(eps)
    return f_hat.float() - e * log_weights(a), g_hat.float() - e * log_weights(b)


def sinkhorn_prelast_potentials_sqeuclid(
    x, y, a, b, *, eps_list: Sequence[float], allow_tf32: bool = False, use_exp2: bool = True,
    autotune: bool = True, block_m=None, block_n=None, block_k=None, num_warps=None, num_stages: int = 2,
    use_flashstyle: Optional[bool] = None, cost_scale: float = 1.0,
    rho_x: Optional[float] = None, rho_y: Optional[float] = None,
):
    """Potentials before the final extrapolation step of a symmetric solve on ``eps_list``."""
    _, _, f_pre, g_pre = sinkhorn_flashstyle_symmetric(
        x, y, a, b, use_epsilon_scaling=False, last_extrapolation=True, allow_tf32=allow_tf32,
        eps_list=eps_list, return_prelast=True, cost_scale=cost_scale, rho_x=rho_x, rho_y=rho_y,
    )
    return f_pre, g_pre


class _PlanSession:
    """Applications of one fixed transport plan through ``fs_plan_session_*``: the clouds are staged and the two
    log-normaliser vectors computed once (two soft-min passes), after which every ``P v``, ``P^T u``, ``P V``,
    ``P^T V``, Mat5 term and CG matvec is a single streaming pass. The reference launches its kernels one call
    at a time (hvp.py:322-594); the pass count per Hessian-vector product is the same (10 + 2K there, 11 + 2K
    here for K CG iterations)."""

    def __init__(self, x, y, f_shift, g_shift, log_a, log_b, *, eps, cost_scale, allow_tf32):
        self.x, self.y = _lib.f32c(x), _lib.f32c(y)
        self.n, self.d = self.x.shape
        self.m = self.y.shape[0]
        self.dev = self.x.device
        self.fh, self.gh = _lib.f32c(f_shift), _lib.f32c(g_shift)
        self.la, self.lb = _lib.f32c(log_a), _lib.f32c(log_b)
        self.eps, self.cs = float(eps), float(cost_scale)
        self.prec = _lib.precision_id(allow_tf32)
        nbytes = int(_lib.load().fs_plan_session_bytes(self.n, self.m, self.d, self.prec))
        self.ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=self.dev)
        _lib.call("fs_plan_session_begin", self.dev, *self._head(), self.eps, self.cs, self.prec, *self._tail())

    def _head(self):
        return (_lib.ptr(self.x), _lib.ptr(self.y), self.n, self.m, self.d, _lib.ptr(self.fh), _lib.ptr(self.gh),
                _lib.ptr(self.la), _lib.ptr(self.lb))

    def _tail(self):
        return (_lib.ptr(self.ws), self.ws.numel(), _lib.stream_ptr(self.dev))

    def _apply(self, kind, operand, dv, scale, coef, out, axis):
        operand = _lib.f32c(operand)
        scale = None if scale is None else _lib.f32c(scale)
        _lib.call("fs_plan_session_apply", self.dev, *self._head(), kind, _lib.ptr(operand), dv, _lib.ptr(scale),
                  float(coef), _lib.ptr(out), axis, self.eps, self.cs, self.prec, *self._tail())
        return out

    def vec(self, v, axis):
        rows = self.n if axis == 1 else self.m
        return self._apply(0, v, 1, None, 1.0, torch.empty((rows,), device=self.dev, dtype=torch.float32), axis)

    def mat(self, V, axis, scale=None):
        rows = self.n if axis == 1 else self.m
        out = torch.empty((rows, V.shape[1]), device=self.dev, dtype=torch.float32)
        return self._apply(1, V, V.shape[1], scale, 1.0, out, axis)

    def mat5(self, A, coef):
        out = torch.empty((self.n, self.d), device=self.dev, dtype=torch.float32)
        return self._apply(2, A, self.d, None, coef, out, 1)

    def schur_cg(self, diag_x, denom, rhs, *, max_iter, rtol, atol):
        z = torch.empty((self.m,), device=self.dev, dtype=torch.float32)
        info = torch.zeros((4,), device=self.dev, dtype=torch.float32)
        dx, dn, rh = _lib.f32c(diag_x), _lib.f32c(denom), _lib.f32c(rhs)
        _lib.call("fs_plan_session_cg", self.dev, *self._head(), _lib.ptr(dx), _lib.ptr(dn), _lib.ptr(rh),
                  _lib.ptr(z), _lib.ptr(info), self.eps, self.cs, int(max_iter), float(rtol), float(atol),
                  self.prec, *self._tail())
        rec = info.tolist()
        _lib.raise_if_device_timeout(self.dev)  # the record read has synchronised: surface a device-side time-out
        return z, CGInfo(bool(rec[0] != 0.0), int(rec[1]), float(rec[2]), float(rec[3]))


def _device_schur_cg(x, y, f_shift, g_shift, log_a, log_b, diag_x, denom, rhs, *, eps, cost_scale,
                     max_iter, rtol, atol, allow_tf32):
    n, d = x.shape
    m = y.shape[0]
    dev = x.device
    prec = _lib.precision_id(allow_tf32)
    z = torch.empty((m,), device=dev, dtype=torch.float32)
    info = torch.zeros((4,), device=dev, dtype=torch.float32)
    ws = _lib.workspace(_lib.OP_SCHUR, n, m, d, prec, dev)
    x32, y32 = _lib.f32c(x), _lib.f32c(y)
    _lib.call(
        "fs_schur_cg", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d,
        _lib.ptr(f_shift), _lib.ptr(g_shift), _lib.ptr(log_a), _lib.ptr(log_b),
        _lib.ptr(_lib.f32c(diag_x)), _lib.ptr(_lib.f32c(denom)), _lib.ptr(_lib.f32c(rhs)),
        _lib.ptr(z), _lib.ptr(info),
        float(eps), float(cost_scale), int(max_iter), float(rtol), float(atol),
        prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    rec = info.tolist()
    _lib.raise_if_device_timeout(dev)  # the record read has synchronised: surface a device-side time-out
    return z, CGInfo(bool(rec[0] != 0.0), int(rec[1]), float(rec[2]), float(rec[3]))


def hvp_x_sqeuclid_from_potentials(
    x: torch.Tensor,
    y: torch.Tensor,
    f_hat: torch.Tensor,
    g_hat: torch.Tensor,
    A: torch.Tensor,
    *,
    eps: float,
    rho_x: Optional[float] = None,
    rho_y: Optional[float] = None,
    cost_scale: float = 1.0,
    lambda_indef: float = 1.0,
    return_components: bool = False,
    tau2: float = 1e-5,
    max_cg_iter: int = 300,
    cg_rtol: float = 1e-6,
    cg_atol: float = 1e-6,
    cg_stabilise_every: int = 0,
    preconditioner: str = "none",
    precond_terms: int = 3,
    use_preconditioner: bool = True,
    allow_tf32: bool = False,
    use_exp2: bool = True,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: int = 4,
    num_stages: int = 2,
    use_fused_matvec: bool = False,
    use_batched_cg: bool = False,
    use_compiled_cg: bool = False,
    use_dense_cg: bool = False,
    autotune: bool = True,
    cg_x0: Optional[torch.Tensor] = None,
):
    """``H @ A`` for the Hessian of the OT cost in x, from OTT-convention potentials.

    ``f_hat, g_hat`` satisfy ``P = exp((f_hat + g_hat - C)/eps)``. Returns ``(hvp, HvpInfo)``,
    or ``(psd_part, indefinite_part, HvpInfo)`` with ``return_components``.
    """
    if x.ndim != 2 or y.ndim != 2 or A.ndim != 2:
        raise ValueError("x,y,A must be 2D tensors.")
    if not x.is_cuda or not y.is_cuda or not f_hat.is_cuda or not g_hat.is_cuda:
        raise ValueError("hvp_x_sqeuclid_from_potentials requires CUDA tensors.")
    n, d = x.shape
    m, d2 = y.shape
    if d != d2 or A.shape != (n, d):
        raise ValueError("Shapes must satisfy x:(n,d), y:(m,d), A:(n,d).")

    mode = str(preconditioner).lower() if use_preconditioner else "none"
    if mode not in ("none", "neumann", "jacobi"):
        raise ValueError("preconditioner must be one of {'none','neumann','jacobi'}.")
    n_terms = int(precond_terms)
    if n_terms < 0:
        raise ValueError("precond_terms must be >= 0.")

    e = float(eps)
    c = 2.0 * cost_scale
    dev = x.device
    xf, yf, Af = x.float(), y.float(), A.float()

    # Shifted potentials in a uniform-weight gauge: the log-weights the kernels add back
    # are subtracted here, so any constant works (reference hvp.py:295-300).
    log_a = torch.full((n,), -math.log(n), device=dev, dtype=torch.float32)
    log_b = torch.full((m,), -math.log(m), device=dev, dtype=torch.float32)
    f_shift = (f_hat.float() - e * log_a - cost_scale * xf.pow(2).sum(dim=1)).contiguous()
    g_shift = (g_hat.float() - e * log_b - cost_scale * yf.pow(2).sum(dim=1)).contiguous()
    # One session for all plan applications below: operands staged once, both normalisers computed once.
    plan = _PlanSession(xf, yf, f_shift, g_shift, log_a, log_b, eps=e, cost_scale=cost_scale, allow_tf32=allow_tf32)

    def P(v):   # [m] -> [n]
        return plan.vec(v, 1)

    def Pt(u):  # [n] -> [m]
        return plan.vec(u, 0)

    def Pmat(V, axis, scale=None):
        return plan.mat(V, axis, scale)

    row_mass = P(torch.ones((m,), device=dev, dtype=torch.float32))
    col_mass = Pt(torch.ones((n,), device=dev, dtype=torch.float32))
    kx = 1.0 if rho_x is None else (float(rho_x) + e) / float(rho_x)
    ky = 1.0 if rho_y is None else (float(rho_y) + e) / float(rho_y)
    floor = max(1e-12, e * 1e-10)
    D_x = kx * row_mass.clamp(min=floor)
    D_y = ky * col_mass.clamp(min=floor)
    balanced = rho_x is None and rho_y is None
    denom = D_y + e * float(tau2) if balanced else D_y

    xa = (x * A).sum(dim=1)                          # x_i . A_i
    Py = Pmat(yf, 1)                                 # [n, d]
    PtA = Pmat(Af, 0)                                # [m, d]
    r_x = c * (row_mass * xa - (A * Py).sum(dim=1))
    r_y = c * (Pt(xa) - (y * PtA).sum(dim=1))
    y1 = r_x / D_x
    rhs_raw = r_y - Pt(y1)

    def schur(zv):
        return denom * zv - Pt(P(zv) / D_x)

    if mode == "none":
        rhs = rhs_raw
        if cg_x0 is None and int(cg_stabilise_every) == 0:
            z, cg = plan.schur_cg(D_x, denom, rhs.contiguous(), max_iter=max_cg_iter, rtol=cg_rtol, atol=cg_atol)
        else:
            z, cg = conjugate_gradient(schur, rhs, x0=cg_x0, max_iter=max_cg_iter, rtol=cg_rtol,
                                       atol=cg_atol, stabilise_every=cg_stabilise_every)
    else:
        def B(zv):
            return Pt(P(zv) / D_x) / denom

        def neumann(v):
            total, term = v, v
            for _ in range(n_terms):
                term = B(term)
                total = total + term
            return total

        z, cg = conjugate_gradient(
            lambda zv: zv - B(zv), rhs_raw / denom, x0=cg_x0, max_iter=max_cg_iter, rtol=cg_rtol,
            atol=cg_atol, preconditioner=neumann if mode == "neumann" else None,
            stabilise_every=cg_stabilise_every,
        )

    Pz = P(z)
    z1 = y1 - Pz / D_x
    Pyz = Pmat(yf, 1, scale=z)
    RTz = c * (x * (row_mass * z1)[:, None] - Py * z1[:, None] + x * Pz[:, None] - Pyz)

    k2 = 2.0 * c / e
    term1 = c * row_mass[:, None] * A
    term2 = -k2 * x * (xa * row_mass)[:, None]
    term3 = k2 * Py * xa[:, None]
    term4 = k2 * x * (Py * A).sum(dim=1)[:, None]
    term5 = plan.mat5(Af, -2.0 * c / e)  # (-4 cs / eps) sum_j P_ij (A_i . y_j) y_j, reference kernels/apply_ott.py:453-566

    psd = RTz / e + term1
    indef = term2 + term3 + term4 + term5
    info = HvpInfo(bool(cg.cg_converged), int(cg.cg_iters), float(cg.cg_residual), float(cg.cg_initial_residual))
    if return_components:
        return psd, indef, info
    return (psd + indef if lambda_indef == 1.0 else psd + lambda_indef * indef), info


def hvp_x_sqeuclid(
    x, y, a, b, A, *, eps_list: Sequence[float], tau2: float = 1e-5, max_cg_iter: int = 300,
    cg_rtol: float = 1e-6, cg_atol: float = 1e-6, cg_stabilise_every: int = 0, preconditioner: str = "none",
    precond_terms: int = 3, use_preconditioner: bool = True, allow_tf32: bool = False, use_exp2: bool = True,
    autotune: bool = True, block_m=None, block_n=None, block_k=None, num_warps=None, num_stages: int = 2,
):
    """Solve for the pre-extrapolation potentials on ``eps_list``, then apply the Hessian to ``A``."""
    eps = float(eps_list[-1])
    f_pre, g_pre = sinkhorn_prelast_potentials_sqeuclid(x, y, a, b, eps_list=eps_list, allow_tf32=allow_tf32)
    f_hat, g_hat = geomloss_to_ott_potentials(f_pre, g_pre, a, b, eps=eps)
    return hvp_x_sqeuclid_from_potentials(
        x, y, f_hat, g_hat, A, eps=eps, tau2=tau2, max_cg_iter=max_cg_iter, cg_rtol=cg_rtol, cg_atol=cg_atol,
        cg_stabilise_every=cg_stabilise_every, preconditioner=preconditioner, precond_terms=precond_terms,
        use_preconditioner=use_preconditioner, allow_tf32=allow_tf32,
    )


def inverse_hvp_x_sqeuclid_from_potentials(
    x: torch.Tensor,
    y: torch.Tensor,
    f_hat: torch.Tensor,
    g_hat: torch.Tensor,
    gr: torch.Tensor,
    *,
    eps: float,
    rho_x: Optional[float] = None,
    rho_y: Optional[float] = None,
    cost_scale: float = 1.0,
    tau2: float = 1e-5,
    max_outer_iter: int = 100,
    outer_rtol: float = 1e-6,
    outer_atol: float = 1e-6,
    max_inner_iter: int = 100,
    inner_rtol: float = 1e-8,
    inner_atol: float = 1e-8,
    cg_stabilise_every: int = 0,
    preconditioner: str = "none",
    precond_terms: int = 3,
    use_preconditioner: bool = True,
    allow_tf32: bool = False,
    use_exp2: bool = True,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: int = 4,
    num_stages: int = 2,
):
    """Solve ``H z = gr`` for the Hessian ``H`` of the OT cost in x (reference hvp.py:696-835).

    Outer conjugate gradients on the flattened ``[n*d]`` vector with :func:`hvp_x_sqeuclid_from_potentials`
    as the operator (whose own Schur-complement solve runs on the device with the ``inner_*`` tolerances).
    Like the reference this assumes ``H`` is positive definite at the given potentials; when it is not, the
    outer loop stops at ``max_outer_iter`` and ``info.cg_converged`` is False. ``cost_scale`` is an extension
    (the reference's inverse solve is fixed to the full squared distance).
    """
    if x.ndim != 2 or y.ndim != 2 or gr.ndim != 2:
        raise ValueError("x, y, gr must be 2D tensors.")
    if not x.is_cuda or not y.is_cuda or not f_hat.is_cuda or not g_hat.is_cuda:
        raise ValueError("inverse_hvp_x_sqeuclid_from_potentials requires CUDA tensors.")
    n, d = x.shape
    m, d2 = y.shape
    if d != d2 or gr.shape != (n, d):
        raise ValueError("Shapes must satisfy x:(n,d), y:(m,d), gr:(n,d).")

    def hessian_times(flat: torch.Tensor) -> torch.Tensor:
        out, _ = hvp_x_sqeuclid_from_potentials(
            x, y, f_hat, g_hat, flat.reshape(n, d), eps=eps, rho_x=rho_x, rho_y=rho_y, cost_scale=cost_scale,
            tau2=tau2, max_cg_iter=max_inner_iter, cg_rtol=inner_rtol, cg_atol=inner_atol,
            cg_stabilise_every=cg_stabilise_every, preconditioner=preconditioner, precond_terms=precond_terms,
            use_preconditioner=use_preconditioner, allow_tf32=allow_tf32,
        )
        return out.reshape(-1)

    z, cg = conjugate_gradient(hessian_times, gr.float().reshape(-1), max_iter=max_outer_iter, rtol=outer_rtol,
                               atol=outer_atol, stabilise_every=cg_stabilise_every)
    info = HvpInfo(bool(cg.cg_converged), int(cg.cg_iters), float(cg.cg_residual), float(cg.cg_initial_residual))
    return z.reshape(n, d), info
