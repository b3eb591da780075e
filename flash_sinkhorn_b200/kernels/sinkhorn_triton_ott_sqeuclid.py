"""OTT-convention primitives kept for import-surface compatibility.

Same names, arguments and return values as the reference's
``kernels/sinkhorn_triton_ott_sqeuclid.py`` (sinkhorn_potentials_sqeuclid :38-148,
apply_lse_kernel_sqeuclid :482-690, update_potential :693-709,
apply_transport_from_potentials_sqeuclid :712-735), with the plan written
``P_ij = exp((f_i + g_j - |x_i - y_j|^2)/eps)``. Nothing here has a kernel of its own: every
function is a short composition of the shifted-potential soft-min pass and the streaming plan
application of the sm_100a engine, so the Triton tuning keywords are accepted and ignored.

How the signed log-sum-exp maps onto the engine. With ``bias_j = (g_j - |y_j|^2)/eps`` the soft-min
pass returns ``-eps*LSE_j[(2/eps) x_i.y_j + bias_j]``, hence

    L_i = eps*log sum_j exp((g_j - C_ij)/eps) = -(pass)_i - |x_i|^2 .

A weight vector ``v`` of either sign is handled without leaving the log domain: the row potential
``-L_i`` makes the plan's rows sum to one, the plan application with that potential returns the
bounded ratio ``r_i = sum_j softmax_ij v_j``, and ``eps*log|sum_j exp(.) v_j| = L_i + eps*log|r_i|``
with the sign of ``r_i``. The row potential ``f_i`` cancels from the reference's result
(it is added inside the exponent and removed afterwards) and is only validated.
"""
from __future__ import annotations

import warnings
from typing import Optional, Tuple

import torch

from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_vec_flashstyle
from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse
from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating

__all__ = [
    "sinkhorn_potentials_sqeuclid",
    "apply_lse_kernel_sqeuclid",
    "update_potential",
    "apply_transport_from_potentials_sqeuclid",
]

# Potentials of masked points may be -inf; the engine's bias must stay finite.
_MASKED = -1.0e30


def sinkhorn_potentials_sqeuclid(
    x: torch.Tensor,
    y: torch.Tensor,
    loga: torch.Tensor,
    logb: torch.Tensor,
    eps: float,
    n_iters: int,
    *,
    fused: bool = True,
    allow_tf32: bool = False,
    use_exp2: bool = True,
    autotune: bool = True,
    cost_scale: float = 1.0,
    rho: Optional[float] = None,
    reach: Optional[float] = None,
    rho_x: Optional[float] = None,
    rho_y: Optional[float] = None,
    reach_x: Optional[float] = None,
    reach_y: Optional[float] = None,
    threshold: Optional[float] = None,
    check_every: int = 5,
    return_n_iters: bool = False,
    **unused,
):
    """Deprecated facade: alternating Sinkhorn with the log-marginals absorbed in the potentials
    (``ott_convention=True`` of :func:`sinkhorn_flashstyle_alternating`)."""
    warnings.warn(
        "sinkhorn_potentials_sqeuclid is deprecated; use sinkhorn_flashstyle_alternating "
        "(flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid) with ott_convention=True.",
        DeprecationWarning, stacklevel=2,
    )
    if unused:
        warnings.warn(f"Unused parameters: {list(unused.keys())}. They are ignored.", UserWarning, stacklevel=2)
    return sinkhorn_flashstyle_alternating(
        x, y, torch.exp(loga), torch.exp(logb), eps=eps, n_iters=n_iters, cost_scale=cost_scale,
        rho=rho, reach=reach, rho_x=rho_x, rho_y=rho_y, reach_x=reach_x, reach_y=reach_y,
        allow_tf32=allow_tf32, threshold=threshold, check_every=check_every,
        return_n_iters=return_n_iters, ott_convention=True,
    )


def _sq_norms(pts: torch.Tensor, given: Optional[torch.Tensor], name: str, count: int) -> torch.Tensor:
    if given is None:
        p32 = pts.float()
        return (p32 * p32).sum(dim=1)
    if given.shape != (count,):
        raise ValueError(f"{name} must have shape ({'n' if name == 'x2' else 'm'},).")
    return given.float()


def apply_lse_kernel_sqeuclid(
    x,
    y,
    f,
    g,
    eps,
    axis,
    vec=None,
    x2=None,
    y2=None,
    block_m=None,
    block_n=None,
    block_k=None,
    num_warps: Optional[int] = None,
    num_stages: Optional[int] = None,
    use_exp2: bool = True,
    allow_tf32: bool = False,
    backend: str = "triton",
    autotune: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``out = eps*log|sum exp((f_i + g_j - C_ij)/eps) * vec| - (f or g)`` and the sign of the sum.

    ``axis=1`` reduces over j (result of length n, ``f`` removed); ``axis=0`` reduces over i (length m,
    ``g`` removed). Without ``vec`` the sign is all ones. A sum that is exactly zero gives ``-inf`` and
    sign 0, as in the reference.
    """
    if not x.is_cuda or not y.is_cuda or not f.is_cuda or not g.is_cuda:
        raise ValueError("apply_lse_kernel_sqeuclid requires CUDA tensors.")
    if x.ndim != 2 or y.ndim != 2:
        raise ValueError("x and y must be 2D tensors.")
    if f.ndim != 1 or g.ndim != 1:
        raise ValueError("f and g must be 1D tensors.")
    if axis not in (0, 1):
        raise ValueError("axis must be 0 or 1.")
    n, d = x.shape
    m, d2 = y.shape
    if d != d2:
        raise ValueError("x and y must have the same feature dimension.")
    if f.shape[0] != n or g.shape[0] != m:
        raise ValueError("f and g shapes must match x and y.")
    if vec is not None:
        if vec.ndim != 1:
            raise ValueError("vec must be a 1D tensor.")
        if axis == 1 and vec.shape[0] != m:
            raise ValueError("vec shape must match axis=1 reduction (m).")
        if axis == 0 and vec.shape[0] != n:
            raise ValueError("vec shape must match axis=0 reduction (n).")
    if backend != "triton":
        raise ValueError(f"Unknown backend={backend!r}. Only 'triton' is supported.")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError(f"Unsupported dtype for x/y: {x.dtype}")
    eps = float(eps)
    xn = _sq_norms(x, x2, "x2", n)
    yn = _sq_norms(y, y2, "y2", m)

    # "rows" keep their index in the result, "cols" are summed over.
    if axis == 1:
        rows, cols, rows2, cols2, col_pot = x, y, xn, yn, g.float()
    else:
        rows, cols, rows2, cols2, col_pot = y, x, yn, xn, f.float()
    col_shift = torch.clamp(col_pot, min=_MASKED) - cols2
    level = -flashsinkhorn_lse(rows, cols, col_shift / eps, eps, allow_tf32=allow_tf32) - rows2
    if vec is None:
        return level, torch.ones_like(level)

    zeros_r = torch.zeros_like(rows2)
    zeros_c = torch.zeros_like(cols2)
    ratio = apply_plan_vec_flashstyle(
        rows, cols, -level - rows2, col_shift, zeros_r, zeros_c, vec.float(),
        eps=eps, axis=1, allow_tf32=allow_tf32,
    )
    mag = ratio.abs()
    out = torch.where(mag > 0, level + eps * torch.log(mag), torch.full_like(level, float("-inf")))
    return out, torch.sign(ratio)


def update_potential(x, y, f, g, log_marginal, eps, axis, **kwargs):
    """One OTT-convention Sinkhorn half-step: ``eps*log_marginal - LSE`` (``axis=1`` updates f,
    ``axis=0`` updates g); non-finite log-sum-exp values count as zero."""
    lse, _ = apply_lse_kernel_sqeuclid(x, y, f, g, eps, axis, **kwargs)
    return eps * log_marginal - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))


def apply_transport_from_potentials_sqeuclid(x, y, f, g, vec, eps, axis, **kwargs):
    """``P @ vec`` (``axis=1``) or ``P.T @ vec`` (``axis=0``) for ``P = exp((f + g - C)/eps)``."""
    lse, sgn = apply_lse_kernel_sqeuclid(x, y, f, g, eps, axis, vec=vec, **kwargs)
    own = f if axis == 1 else g
    return sgn * torch.exp((lse + own) / float(eps))
