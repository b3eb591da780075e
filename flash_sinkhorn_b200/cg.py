"""Conjugate gradient for symmetric positive (semi-)definite operators.

``conjugate_gradient`` / ``CGInfo`` follow the reference's ``cg.py:19-121``: same
stopping rule (``|r| <= max(atol, rtol*|r0|)``), same bookkeeping (``cg_iters`` is
``max_iter`` when the tolerance was not reached). This host-driven version takes an
arbitrary ``matvec`` callable and synchronises once per iteration; the HVP's default
path uses the device-resident loop ``fs_schur_cg`` instead (see ``hvp.py``).

``steihaug_cg`` / ``SteihaugCGInfo`` (reference ``cg.py:129-369``) solve the trust-region
subproblem ``min g.p + p.H.p/2, |p| <= delta`` by truncated CG (Steihaug 1983; Nocedal & Wright,
Algorithm 7.2): host-driven as well, one Hessian-vector callable, 1-D tensors.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch

__all__ = ["CGInfo", "conjugate_gradient", "SteihaugCGInfo", "steihaug_cg"]


@dataclass(frozen=True)
class CGInfo:
    cg_converged: bool
    cg_iters: int
    cg_residual: float
    cg_initial_residual: float


def conjugate_gradient(
    matvec: Callable[[torch.Tensor], torch.Tensor],
    b: torch.Tensor,
    *,
    x0: Optional[torch.Tensor] = None,
    max_iter: int = 300,
    rtol: float = 1e-6,
    atol: float = 1e-6,
    preconditioner: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
    stabilise_every: int = 0,
) -> Tuple[torch.Tensor, CGInfo]:
    """Solve ``A x = b`` for a symmetric positive definite ``A`` given as ``matvec``."""
    every = int(stabilise_every)
    if every < 0:
        raise ValueError("stabilise_every must be >= 0.")
    apply_m = preconditioner if preconditioner is not None else (lambda v: v)

    if x0 is None:
        sol = torch.zeros_like(b)
        resid = b.clone()
    else:
        sol = x0.clone()
        resid = b - matvec(sol)
    zvec = apply_m(resid)
    direction = zvec.clone()
    rz = torch.dot(resid, zvec)
    r0 = float(torch.linalg.norm(resid))
    tol = max(atol, rtol * r0)

    for k in range(int(max_iter)):
        a_dir = matvec(direction)
        curv = torch.dot(direction, a_dir)
        if curv.abs() == 0:
            break
        step = rz / curv
        sol = sol + step * direction
        resid = resid - step * a_dir
        if every and (k + 1) % every == 0:
            resid = b - matvec(sol)
        rnorm = float(torch.linalg.norm(resid))
        if rnorm <= tol:
            return sol, CGInfo(True, k + 1, rnorm, r0)
        zvec = apply_m(resid)
        rz_next = torch.dot(resid, zvec)
        direction = zvec + (rz_next / rz) * direction
        rz = rz_next

    return sol, CGInfo(False, int(max_iter), float(torch.linalg.norm(resid)), r0)


@dataclass(frozen=True)
class SteihaugCGInfo:
    """Outcome of :func:`steihaug_cg`. ``termination_reason`` is one of ``"converged"`` (residual below
    tolerance inside the region), ``"negative_curvature"`` (``d.H.d <= neg_curv_tol``: followed ``d`` to the
    boundary), ``"boundary"`` (the CG step left the region and was cut there) or ``"max_iter"``."""

    converged: bool
    iters: int
    residual: float
    termination_reason: str
    hit_boundary: bool
    negative_curvature_detected: bool
    predicted_reduction: float


def _step_to_boundary(point: torch.Tensor, direction: torch.Tensor, delta: float) -> float:
    """``tau > 0`` with ``|point + tau*direction| = delta`` (forward intersection with the sphere)."""
    pp = float(torch.dot(point, point))
    pd = float(torch.dot(point, direction))
    dd = float(torch.dot(direction, direction))
    # dd*tau^2 + 2*pd*tau + (pp - delta^2) = 0
    quarter_disc = pd * pd - dd * (pp - delta * delta)
    if quarter_disc < 0.0:  # only possible when the point is already outside
        return delta / math.sqrt(dd + 1e-10)
    root = math.sqrt(quarter_disc)
    denom = dd + 0.5e-10
    forward, backward = (-pd + root) / denom, (-pd - root) / denom
    positive = [t for t in (forward, backward) if t > 0]
    return min(positive) if positive else abs(forward)


def steihaug_cg(
    hvp_fn: Callable[[torch.Tensor], torch.Tensor],
    grad: torch.Tensor,
    delta: float,
    *,
    max_iter: int = 100,
    rtol: float = 1e-6,
    atol: float = 1e-6,
    neg_curv_tol: float = 1e-10,
) -> Tuple[torch.Tensor, SteihaugCGInfo]:
    """Approximate minimiser of ``grad.p + p.H.p/2`` over ``|p| <= delta``; ``H`` may be indefinite.

    CG on ``H p = -grad`` from ``p = 0``. The first direction of non-positive curvature, or the first step
    that would leave the region, is followed exactly to the boundary and returned. ``predicted_reduction``
    is ``-(grad.p + p.H.p/2)`` of the returned step (one extra Hessian-vector product).
    """

    def finish(step, reason, iters, resid, neg):
        h_step = hvp_fn(step)
        reduction = -float(torch.dot(grad, step)) - 0.5 * float(torch.dot(step, h_step))
        on_boundary = reason in ("negative_curvature", "boundary")
        if reason == "max_iter":
            on_boundary = float(torch.linalg.norm(step)) >= 0.99 * delta
        return step, SteihaugCGInfo(reason == "converged", iters, resid, reason, on_boundary, neg, reduction)

    step = torch.zeros_like(grad)
    resid = -grad.clone()
    direction = resid.clone()
    rnorm = float(torch.linalg.norm(resid))
    tol = max(atol, rtol * rnorm)
    if rnorm < tol:
        return step, SteihaugCGInfo(True, 0, rnorm, "converged", False, False, 0.0)

    for k in range(int(max_iter)):
        h_dir = hvp_fn(direction)
        curv = float(torch.dot(direction, h_dir))
        if curv <= neg_curv_tol:
            tau = _step_to_boundary(step, direction, delta)
            return finish(step + tau * direction, "negative_curvature", k + 1, rnorm, True)
        rr = float(torch.dot(resid, resid))
        length = rr / curv
        trial = step + length * direction
        if float(torch.linalg.norm(trial)) >= delta:
            tau = _step_to_boundary(step, direction, delta)
            return finish(step + tau * direction, "boundary", k + 1, rnorm, False)
        step = trial
        resid = resid - length * h_dir
        rnorm = float(torch.linalg.norm(resid))
        if rnorm < tol:
            return finish(step, "converged", k + 1, rnorm, False)
        direction = resid + (float(torch.dot(resid, resid)) / rr) * direction

    return finish(step, "max_iter", int(max_iter), rnorm, False)
