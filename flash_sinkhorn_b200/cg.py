"""Conjugate gradient for symmetric positive (semi-)definite operators.

``conjugate_gradient`` / ``CGInfo`` follow the reference's ``cg.py:19-121``: same
stopping rule (``|r| <= max(atol, rtol*|r0|)``), same bookkeeping (``cg_iters`` is
``max_iter`` when the tolerance was not reached). This host-driven version takes an
arbitrary ``matvec`` callable and synchronises once per iteration; the HVP's default
path uses the device-resident loop ``fs_schur_cg`` instead (see ``hvp.py``).
The reference's trust-region ``steihaug_cg`` is not provided.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch

__all__ = ["CGInfo", "conjugate_gradient"]


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
