"""Implicit differentiation through the Sinkhorn fixed point (gradient w.r.t. the source cloud).

API and semantics follow the reference's ``implicit_grad.py`` (``ImplicitGradInfo`` :29-33,
``implicit_grad_x_from_potentials`` :36-242, ``implicit_grad_x`` :245-315).

At a converged plan ``P`` with marginals ``r = P 1``, ``c = P^T 1`` the optimality conditions
``F(f, g; x) = (r - a, c - b) = 0`` define the potentials implicitly. For a loss with gradients
``(grad_f, grad_g)`` w.r.t. the potentials, the multipliers solve the symmetric system

    [ diag(r)  P       ] [lam_f]         [grad_f]
    [ P^T      diag(c) ] [lam_g] = eps * [grad_g]

which is reduced to its Schur complement in ``lam_g`` (Tikhonov term ``eps*tau2`` on the diagonal) and
solved by conjugate gradients; the result is pushed through ``dF/dx``. Every product with ``P`` streams
through the CUDA engine (``apply_plan_vec/mat_flashstyle``) and the CG loop itself runs on the device
(``fs_schur_cg``: no host synchronisation per iteration), unlike the reference's host-driven loop.
"""
from __future__ import annotations

import math
import warnings
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from flash_sinkhorn_b200.hvp import _device_schur_cg
from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle

__all__ = ["ImplicitGradInfo", "implicit_grad_x_from_potentials", "implicit_grad_x"]


@dataclass(frozen=True)
class ImplicitGradInfo:
    cg_converged: bool
    cg_iters: int
    cg_residual: float


def implicit_grad_x_from_potentials(
    x: torch.Tensor,
    y: torch.Tensor,
    f_hat: torch.Tensor,
    g_hat: torch.Tensor,
    grad_f: torch.Tensor,
    grad_g: torch.Tensor,
    *,
    eps: float,
    log_a: Optional[torch.Tensor] = None,
    log_b: Optional[torch.Tensor] = None,
    cost_scale: float = 1.0,
    tau2: float = 1e-5,
    max_cg_iter: int = 100,
    cg_rtol: float = 1e-6,
    cg_atol: float = 1e-6,
    allow_tf32: bool = False,
    use_exp2: bool = True,
) -> Tuple[torch.Tensor, ImplicitGradInfo]:
    """``dL/dx`` ([n, d]) from shifted potentials ``f_hat = f - cs|x|^2``, ``g_hat = g - cs|y|^2`` and the
    loss gradients w.r.t. the potentials. Missing log-weights default to uniform marginals."""
    if x.ndim != 2 or y.ndim != 2:
        raise ValueError("x, y must be 2D tensors.")
    if not x.is_cuda:
        raise ValueError("CUDA required.")
    n, _ = x.shape
    m = y.shape[0]
    e = float(eps)
    dev = x.device
    if log_a is None:
        log_a = torch.full((n,), -math.log(n), device=dev, dtype=torch.float32)
    if log_b is None:
        log_b = torch.full((m,), -math.log(m), device=dev, dtype=torch.float32)
    fh, gh = f_hat.float().contiguous(), g_hat.float().contiguous()
    la, lb = log_a.float().contiguous(), log_b.float().contiguous()
    gf, gg = grad_f.float(), grad_g.float()
    xf, yf = x.float(), y.float()
    kw = dict(eps=e, cost_scale=cost_scale, allow_tf32=allow_tf32)

    def plan_vec(v, axis):
        return apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, v, axis=axis, **kw)

    def plan_rows(mat, scale=None):
        return apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, mat, axis=1, scale=scale, **kw)

    row_mass = plan_vec(torch.ones((m,), device=dev, dtype=torch.float32), 1)
    col_mass = plan_vec(torch.ones((n,), device=dev, dtype=torch.float32), 0)

    # Schur complement in lam_g, multiplied through by eps so that it has the engine's form
    #   (diag(c + eps*tau2) - P^T diag(1/r) P) lam_g = eps * (grad_g - P^T (grad_f / r)).
    # CG is invariant under that scaling; the absolute tolerance and the reported residual are scaled back.
    rhs = e * (gg - plan_vec(gf / row_mass, 0))
    lam_g, cg = _device_schur_cg(
        x, y, fh, gh, la, lb, row_mass, col_mass + e * float(tau2), rhs.contiguous(), eps=e,
        cost_scale=cost_scale, max_iter=int(max_cg_iter), rtol=float(cg_rtol), atol=e * float(cg_atol),
        allow_tf32=allow_tf32,
    )
    plan_lam_g = plan_vec(lam_g, 1)
    lam_f = (e * gf - plan_lam_g) / row_mass

    # dL/dx_i = (2/eps) [ lam_f_i (r_i x_i - (P y)_i) + (P lam_g)_i x_i - (P (lam_g * y))_i ]
    plan_y = plan_rows(yf)
    plan_y_weighted = plan_rows(yf, scale=lam_g)
    bracket = lam_f[:, None] * (xf * row_mass[:, None] - plan_y) + plan_lam_g[:, None] * xf - plan_y_weighted
    grad_x = (2.0 / e) * bracket
    return grad_x, ImplicitGradInfo(bool(cg.cg_converged), int(cg.cg_iters), float(cg.cg_residual) / e)


def implicit_grad_x(
    x: torch.Tensor,
    y: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    grad_f: torch.Tensor,
    grad_g: torch.Tensor,
    *,
    eps: float,
    cost_scale: float = 1.0,
    n_iters: int = 100,
    tau2: float = 1e-5,
    max_cg_iter: int = 100,
    cg_rtol: float = 1e-6,
    cg_atol: float = 1e-6,
    allow_tf32: bool = False,
    use_exp2: bool = True,
    autotune: bool = True,
    use_flashstyle: Optional[bool] = None,
) -> Tuple[torch.Tensor, ImplicitGradInfo]:
    """Solve the symmetric Sinkhorn problem at fixed ``eps`` (``n_iters`` steps plus extrapolation), then
    differentiate implicitly. ``use_flashstyle=False`` only warns, as in the reference."""
    if use_flashstyle is not None and not use_flashstyle:
        warnings.warn("use_flashstyle=False is deprecated. FlashSinkhorn is now the only backend.",
                      DeprecationWarning, stacklevel=2)
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric

    f, g = sinkhorn_flashstyle_symmetric(
        x, y, a, b, use_epsilon_scaling=False, eps=eps, cost_scale=cost_scale, n_iters=n_iters,
        last_extrapolation=True, allow_tf32=allow_tf32,
    )
    f_hat = f - cost_scale * x.float().pow(2).sum(dim=1)
    g_hat = g - cost_scale * y.float().pow(2).sum(dim=1)
    return implicit_grad_x_from_potentials(
        x, y, f_hat, g_hat, grad_f, grad_g, eps=eps, log_a=torch.log(a.float().clamp(min=1e-20)),
        log_b=torch.log(b.float().clamp(min=1e-20)), cost_scale=cost_scale, tau2=tau2,
        max_cg_iter=max_cg_iter, cg_rtol=cg_rtol, cg_atol=cg_atol, allow_tf32=allow_tf32,
    )
