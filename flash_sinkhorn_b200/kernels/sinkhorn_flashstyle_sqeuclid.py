"""Shifted-potential log-sum-exp updates: Python launchers over the CUDA engine.

Same call signatures as the reference's ``kernels/sinkhorn_flashstyle_sqeuclid.py``
(flashsinkhorn_lse :815-955, flashsinkhorn_lse_fused :958-1090,
flashsinkhorn_symmetric_step :1093-1317, helpers :68-147 and :1324-1363). The Triton
tuning keywords (``block_*``, ``num_warps``, ``num_stages``, ``autotune``, ``use_exp2``)
are accepted for compatibility and ignored: tiling is fixed inside the sm_100a kernels
and the exponentials are always evaluated in base 2.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from flash_sinkhorn_b200 import _lib
from flash_sinkhorn_b200.kernels._common import log_weights


def precompute_flashsinkhorn_inputs(
    x: torch.Tensor, y: torch.Tensor, a: torch.Tensor, b: torch.Tensor, eps: float, cost_scale: float = 1.0
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(alpha, beta, gamma, delta)`` = ``(cs|x|^2, cs|y|^2, eps*log a, eps*log b)``."""
    alpha = cost_scale * x.float().pow(2).sum(dim=1)
    beta = cost_scale * y.float().pow(2).sum(dim=1)
    return alpha, beta, eps * log_weights(a), eps * log_weights(b)


def compute_bias_f(g: torch.Tensor, beta: torch.Tensor, delta: torch.Tensor, eps: float) -> torch.Tensor:
    """Pre-scaled column bias of the f-update: ``(g - beta + delta)/eps``."""
    return ((g - beta) + delta) / eps


def compute_bias_g(f: torch.Tensor, alpha: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """Pre-scaled column bias of the g-update: ``(f - alpha + gamma)/eps``."""
    return ((f - alpha) + gamma) / eps


def shifted_to_standard_potentials(f_hat, g_hat, alpha, beta):
    return f_hat + alpha, g_hat + beta


def standard_to_shifted_potentials(f, g, alpha, beta):
    return f - alpha, g - beta


def _check_clouds(x: torch.Tensor, y: torch.Tensor) -> Tuple[int, int, int]:
    if not x.is_cuda or not y.is_cuda:
        raise ValueError("x and y must be CUDA tensors")
    if x.ndim != 2 or y.ndim != 2:
        raise ValueError("x and y must be 2D tensors")
    n, d = x.shape
    m, d2 = y.shape
    if d != d2:
        raise ValueError("x and y must have same feature dimension")
    return n, m, d


def _lse_call(x, y, pot, logw, eps, cost_scale, damping, allow_tf32) -> torch.Tensor:
    n, m, d = _check_clouds(x, y)
    dev = _lib.require_cuda(x=x, y=y, bias=pot, log_w=logw)
    x32, y32, pot32 = _lib.f32c(x), _lib.f32c(y), _lib.f32c(pot)
    logw32 = None if logw is None else _lib.f32c(logw)
    prec = _lib.precision_id(allow_tf32)
    out = torch.empty((n,), device=dev, dtype=torch.float32)
    ws = _lib.workspace(_lib.OP_LSE, n, m, d, prec, dev)
    _lib.call(
        "fs_lse", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d, _lib.ptr(pot32), _lib.ptr(logw32), _lib.ptr(out),
        float(eps), float(cost_scale), float(damping), prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    return out


def flashsinkhorn_lse(
    x: torch.Tensor,
    y: torch.Tensor,
    bias: torch.Tensor,
    eps: float,
    *,
    cost_scale: float = 1.0,
    damping: float = 1.0,
    allow_tf32: bool = True,
    use_exp2: bool = True,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: Optional[int] = None,
    num_stages: int = 2,
    autotune: bool = True,
) -> torch.Tensor:
    """``out_i = -eps*damping*LSE_j[(2*cost_scale/eps) x_i.y_j + bias_j]`` with a pre-scaled bias."""
    if bias.ndim != 1:
        raise ValueError("bias must be 1D tensor")
    if x.ndim == 2 and y.ndim == 2 and bias.shape[0] != y.shape[0]:
        raise ValueError(f"bias must have length {y.shape[0]}, got {bias.shape[0]}")
    return _lse_call(x, y, bias, None, eps, cost_scale, damping, allow_tf32)


def flashsinkhorn_lse_fused(
    x: torch.Tensor,
    y: torch.Tensor,
    g_hat: torch.Tensor,
    log_w: torch.Tensor,
    eps: float,
    *,
    cost_scale: float = 1.0,
    damping: float = 1.0,
    allow_tf32: bool = True,
    use_exp2: bool = True,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: Optional[int] = None,
    num_stages: int = 2,
    autotune: bool = True,
) -> torch.Tensor:
    """Same update with the bias ``g_hat/eps + log_w`` formed inside the kernel."""
    if g_hat.ndim != 1 or log_w.ndim != 1:
        raise ValueError("g_hat and log_w must be 1D tensors")
    if x.ndim == 2 and y.ndim == 2:
        m = y.shape[0]
        if g_hat.shape[0] != m:
            raise ValueError(f"g_hat must have length {m}, got {g_hat.shape[0]}")
        if log_w.shape[0] != m:
            raise ValueError(f"log_w must have length {m}, got {log_w.shape[0]}")
    return _lse_call(x, y, g_hat, log_w, eps, cost_scale, damping, allow_tf32)


def flashsinkhorn_symmetric_step(
    x: torch.Tensor,
    y: torch.Tensor,
    f_hat: torch.Tensor,
    g_hat: torch.Tensor,
    log_a: torch.Tensor,
    log_b: torch.Tensor,
    eps: float,
    *,
    cost_scale: float = 1.0,
    alpha: float = 0.5,
    damping_f: float = 1.0,
    damping_g: float = 1.0,
    allow_tf32: bool = True,
    use_exp2: bool = True,
    autotune: bool = True,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: Optional[int] = None,
    num_stages: int = 2,
    label_x: Optional[torch.Tensor] = None,
    label_y: Optional[torch.Tensor] = None,
    label_cost_matrix: Optional[torch.Tensor] = None,
    lambda_x: float = 1.0,
    lambda_y: float = 0.0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """One Jacobi step on both potentials: ``new = (1-alpha)*old + alpha*candidate``.

    Both candidates are computed from the old potentials. The unbalanced shift
    correction is NOT applied here (as in the reference, the solver does it).
    """
    n, d = x.shape
    m = y.shape[0]
    dev = _lib.require_cuda(x=x, y=y, f_hat=f_hat, g_hat=g_hat, log_a=log_a, log_b=log_b)
    labels = _lib.LabelCost.make(label_x, label_y, label_cost_matrix, lambda_x, lambda_y, n, m, dev)
    x32, y32 = _lib.f32c(x), _lib.f32c(y)
    f32, g32, la32, lb32 = _lib.f32c(f_hat), _lib.f32c(g_hat), _lib.f32c(log_a), _lib.f32c(log_b)
    prec = _lib.precision_id(allow_tf32)
    f_out = torch.empty((n,), device=dev, dtype=torch.float32)
    g_out = torch.empty((m,), device=dev, dtype=torch.float32)
    ws = _lib.workspace(_lib.OP_STEP, n, m, d, prec, dev, labels.V if labels else 0)
    _lib.call(
        "fs_symmetric_step", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d,
        _lib.ptr(f32), _lib.ptr(g32), _lib.ptr(la32), _lib.ptr(lb32),
        _lib.ptr(f_out), _lib.ptr(g_out), None, None,
        float(eps), float(alpha), float(damping_f), float(damping_g), float(cost_scale),
        prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev), labels.ref if labels else None,
    )
    return f_out, g_out


# Solver loops live in flash_sinkhorn_b200.sinkhorn_solvers; re-exported here because the
# reference exposes them from this module path too.
from flash_sinkhorn_b200.sinkhorn_solvers import (  # noqa: E402,F401
    sinkhorn_flashstyle_alternating,
    sinkhorn_flashstyle_symmetric,
)
