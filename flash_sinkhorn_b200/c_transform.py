"""Hard (non-entropic) Kantorovich c-transform and the differentiable semi-dual objective.

Public surface of the reference's ``c_transform.py`` (``c_transform_fwd`` :32-112,
``_CTransformCostFunction`` :115-174, ``c_transform_cost`` :177-241):

    c^psi(x_i) = min_j [ cost_scale*|x_i - y_j|^2 - psi_j ],     j*(i) = arg min (smallest j on ties)
    L(x, psi)  = sum_i a_i c^psi(x_i) + sum_j b_j psi_j

with the Danskin gradients ``dL/dx_i = a_i 2 cs (x_i - y_{j*(i)})`` and ``dL/dpsi_j = b_j - sum_{i: j*(i)=j} a_i``.
The n x m search runs in the CUDA engine (``kernels.c_transform_sqeuclid``); gather / scatter of the matched
points are O(n d) torch ops.
"""
from __future__ import annotations

from typing import Optional

import torch

from flash_sinkhorn_b200.kernels.c_transform_sqeuclid import c_transform_kernel

__all__ = ["c_transform_fwd", "c_transform_cost"]


def _same_device(ref: torch.Tensor, **others: torch.Tensor) -> None:
    for name, t in others.items():
        if not t.is_cuda or t.device != ref.device:
            raise ValueError(f"{name} must be on the same CUDA device as x ({ref.device}), got {t.device}")


def c_transform_fwd(x, y, psi, *, cost_scale: float = 1.0, allow_tf32: bool = True, autotune: bool = True,
                    **kernel_kwargs):
    """``(c_values [n] float32, argmin_idx [n] int64)``, detached (building block, not differentiable)."""
    if x.ndim != 2:
        raise ValueError(f"x must be 2D [n, d], got shape {x.shape}")
    if y.ndim != 2:
        raise ValueError(f"y must be 2D [m, d], got shape {y.shape}")
    if psi.ndim != 1:
        raise ValueError(f"psi must be 1D [m], got shape {psi.shape}")
    d, (m, d2) = x.shape[1], y.shape
    if d != d2:
        raise ValueError(f"x and y must have same feature dim, got {d} vs {d2}")
    if psi.shape[0] != m:
        raise ValueError(f"psi must have length {m}, got {psi.shape[0]}")
    if m == 0:
        raise ValueError("m must be > 0")
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor")
    _same_device(x, y=y, psi=psi)
    if y.requires_grad:
        raise NotImplementedError("grad_y not supported for c_transform_fwd. "
                                  "Detach y or use a solver that supports grad_y.")
    yf, xf = y.detach().float(), x.detach().float()
    bias = cost_scale * (yf * yf).sum(dim=1) - psi.detach().float()
    inner, idx = c_transform_kernel(xf, yf, bias, cost_scale=cost_scale, allow_tf32=allow_tf32, autotune=autotune,
                                    **kernel_kwargs)
    return (cost_scale * (xf * xf).sum(dim=1) + inner).detach(), idx.detach()


class _CTransformCostFunction(torch.autograd.Function):
    """Semi-dual objective; backward by Danskin's theorem at the stored arg-min."""

    @staticmethod
    def forward(ctx, x, y, psi, cost_scale, allow_tf32, autotune, a, b):
        c_values, idx = c_transform_fwd(x, y, psi, cost_scale=cost_scale, allow_tf32=allow_tf32, autotune=autotune)
        ctx.save_for_backward(x, y, idx, a, b)
        ctx.cost_scale = cost_scale
        return (a * c_values).sum() + (b * psi.float()).sum()

    @staticmethod
    def backward(ctx, grad_output):
        x, y, idx, a, b = ctx.saved_tensors
        if ctx.needs_input_grad[1]:
            raise NotImplementedError("grad_y not implemented for c_transform_cost. "
                                      "Detach y before passing to c_transform_cost.")
        grad_x = grad_psi = None
        if ctx.needs_input_grad[0]:
            grad_x = grad_output * (a * (2.0 * ctx.cost_scale)).unsqueeze(1) * (x.float() - y.float()[idx])
        if ctx.needs_input_grad[2]:
            mass = torch.zeros(y.shape[0], device=a.device, dtype=torch.float32)
            mass.scatter_add_(0, idx, a)
            grad_psi = grad_output * (b - mass)
        return grad_x, None, grad_psi, None, None, None, None, None


def c_transform_cost(x, y, psi, *, cost_scale: float = 1.0, allow_tf32: bool = True, autotune: bool = True,
                     a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Scalar ``L(x, psi)``, differentiable w.r.t. x and psi (not y; weights must not require grad)."""
    n, m = x.shape[0], y.shape[0]
    if a is None:
        a = torch.full((n,), 1.0 / n, device=x.device, dtype=torch.float32)
    if b is None:
        b = torch.full((m,), 1.0 / m, device=y.device, dtype=torch.float32)
    if a.shape != (n,):
        raise ValueError(f"a must have shape ({n},), got {a.shape}")
    if b.shape != (m,):
        raise ValueError(f"b must have shape ({m},), got {b.shape}")
    _same_device(x, a=a, b=b)
    if a.requires_grad:
        raise ValueError("a must not require grad (weights are non-differentiable)")
    if b.requires_grad:
        raise ValueError("b must not require grad (weights are non-differentiable)")
    return _CTransformCostFunction.apply(x, y, psi, cost_scale, allow_tf32, autotune, a.float(), b.float())
