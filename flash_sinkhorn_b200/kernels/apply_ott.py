"""Operations on OTT-convention potentials, ``P_ij = exp((f_i + g_j - cost_scale*C_ij)/eps)``.

``mat5_sqeuclid`` has the signature of the reference's ``kernels/apply_ott.py:453-566``:
``out_i = (-4*cost_scale/eps) * sum_j P_ij (A_i . y_j) y_j``.
``apply_plan_vec_sqeuclid`` / ``apply_plan_mat_sqeuclid`` (reference :213-450) are the deprecated
OTT-convention spellings of the plan applications: they subtract ``eps*log w`` and the squared
norms from the potentials and forward to the shifted-potential entry points.
"""
from __future__ import annotations

import math
import warnings
from typing import Optional

import torch

from flash_sinkhorn_b200 import _lib
from flash_sinkhorn_b200.kernels._common import validate_device


def _ott_to_shifted(x, y, f, g, eps, cost_scale, log_a, log_b):
    """OTT-convention ``(f, g)`` -> shifted potentials and the log-weights they go with.

    ``f = f_std + eps*log a`` and ``f_hat = f_std - cost_scale*|x|^2`` give
    ``f_hat = f - eps*log a - cost_scale*|x|^2``; missing log-weights mean uniform weights.
    """
    n, m = x.shape[0], y.shape[0]
    if log_a is None:
        log_a = torch.full((n,), -math.log(n), device=x.device, dtype=torch.float32)
    if log_b is None:
        log_b = torch.full((m,), -math.log(m), device=x.device, dtype=torch.float32)
    f_hat = f.float() - eps * log_a - cost_scale * x.float().pow(2).sum(dim=1)
    g_hat = g.float() - eps * log_b - cost_scale * y.float().pow(2).sum(dim=1)
    return f_hat, g_hat, log_a, log_b


def _check_ott_args(x, y, f, g, axis):
    if axis not in (0, 1):
        raise ValueError("axis must be 0 or 1.")
    if not x.is_cuda:
        raise ValueError("CUDA required.")
    if f.ndim != 1 or g.ndim != 1:
        raise ValueError("f and g must be 1D.")


def apply_plan_vec_sqeuclid(
    x: torch.Tensor,
    y: torch.Tensor,
    f: torch.Tensor,
    g: torch.Tensor,
    vec: torch.Tensor,
    *,
    eps: float,
    axis: int,
    cost_scale: float = 1.0,
    x2: Optional[torch.Tensor] = None,
    y2: Optional[torch.Tensor] = None,
    log_a: Optional[torch.Tensor] = None,
    log_b: Optional[torch.Tensor] = None,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: int = 4,
    num_stages: int = 2,
    use_exp2: bool = True,
    allow_tf32: bool = False,
    autotune: bool = True,
) -> torch.Tensor:
    """Deprecated. ``out_i = sum_j P_ij vec_j`` (``axis=1``) or ``out_j = sum_i P_ij vec_i`` (``axis=0``)."""
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_vec_flashstyle

    warnings.warn(
        "apply_plan_vec_sqeuclid is deprecated; use apply_plan_vec_flashstyle with shifted potentials.",
        DeprecationWarning, stacklevel=2,
    )
    _check_ott_args(x, y, f, g, axis)
    if x.ndim != 2 or y.ndim != 2:
        raise ValueError("x and y must be (n,d) and (m,d).")
    if vec.ndim != 1:
        raise ValueError("vec must be 1D.")
    validate_device(x, [("y", y), ("f", f), ("g", g), ("vec", vec), ("x2", x2), ("y2", y2)])
    n, d = x.shape
    m, d2 = y.shape
    if d != d2:
        raise ValueError("x and y must have the same feature dimension.")
    if f.shape[0] != n or g.shape[0] != m:
        raise ValueError("f and g shapes must match x and y.")
    if axis == 1 and vec.shape[0] != m:
        raise ValueError("vec must have shape (m,) for axis=1.")
    if axis == 0 and vec.shape[0] != n:
        raise ValueError("vec must have shape (n,) for axis=0.")
    f_hat, g_hat, log_a, log_b = _ott_to_shifted(x, y, f, g, eps, cost_scale, log_a, log_b)
    return apply_plan_vec_flashstyle(x, y, f_hat, g_hat, log_a, log_b, vec, eps=eps, axis=axis,
                                     cost_scale=cost_scale, allow_tf32=allow_tf32)


def apply_plan_mat_sqeuclid(
    x: torch.Tensor,
    y: torch.Tensor,
    f: torch.Tensor,
    g: torch.Tensor,
    mat: torch.Tensor,
    *,
    eps: float,
    axis: int,
    cost_scale: float = 1.0,
    scale: Optional[torch.Tensor] = None,
    x2: Optional[torch.Tensor] = None,
    y2: Optional[torch.Tensor] = None,
    log_a: Optional[torch.Tensor] = None,
    log_b: Optional[torch.Tensor] = None,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    block_d: Optional[int] = None,
    num_warps: int = 4,
    num_stages: int = 2,
    use_exp2: bool = True,
    allow_tf32: bool = False,
    autotune: bool = True,
) -> torch.Tensor:
    """Deprecated. ``P @ mat`` (``axis=1``, optional per-column ``scale``) or ``P.T @ mat`` (``axis=0``)."""
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle

    warnings.warn(
        "apply_plan_mat_sqeuclid is deprecated; use apply_plan_mat_flashstyle with shifted potentials.",
        DeprecationWarning, stacklevel=2,
    )
    _check_ott_args(x, y, f, g, axis)
    if x.ndim != 2 or y.ndim != 2 or mat.ndim != 2:
        raise ValueError("x,y,mat must be 2D tensors.")
    validate_device(x, [("y", y), ("f", f), ("g", g), ("mat", mat), ("scale", scale), ("x2", x2), ("y2", y2)])
    n, d = x.shape
    m, d2 = y.shape
    if d != d2:
        raise ValueError("x and y must have the same feature dimension.")
    if f.shape[0] != n or g.shape[0] != m:
        raise ValueError("f and g shapes must match x and y.")
    if axis == 1 and mat.shape != (m, d):
        raise ValueError("For axis=1, mat must have shape (m, d).")
    if axis == 0 and mat.shape != (n, d):
        raise ValueError("For axis=0, mat must have shape (n, d).")
    if scale is not None:
        if axis != 1:
            raise ValueError("scale is only supported for axis=1.")
        if scale.shape != (m,):
            raise ValueError("scale must have shape (m,).")
    f_hat, g_hat, log_a, log_b = _ott_to_shifted(x, y, f, g, eps, cost_scale, log_a, log_b)
    return apply_plan_mat_flashstyle(x, y, f_hat, g_hat, log_a, log_b, mat, eps=eps, axis=axis,
                                     cost_scale=cost_scale, scale=scale, allow_tf32=allow_tf32)


def mat5_sqeuclid(
    x: torch.Tensor,
    y: torch.Tensor,
    f: torch.Tensor,
    g: torch.Tensor,
    A: torch.Tensor,
    *,
    eps: float,
    cost_scale: float = 1.0,
    x2: Optional[torch.Tensor] = None,
    y2: Optional[torch.Tensor] = None,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: int = 4,
    num_stages: int = 2,
    use_exp2: bool = True,
    allow_tf32: bool = False,
    autotune: bool = True,
) -> torch.Tensor:
    if not x.is_cuda:
        raise ValueError("CUDA required.")
    if x.ndim != 2 or y.ndim != 2 or A.ndim != 2:
        raise ValueError("x,y,A must be 2D tensors.")
    validate_device(x, [("y", y), ("f", f), ("g", g), ("A", A), ("x2", x2), ("y2", y2)])
    n, d = x.shape
    m, d2 = y.shape
    if d != d2 or A.shape != (n, d):
        raise ValueError("Shapes must satisfy x:(n,d), y:(m,d), A:(n,d).")
    dev = x.device
    x32, y32, f32, g32, A32 = map(_lib.f32c, (x, y, f, g, A))
    prec = _lib.precision_id(allow_tf32)
    out = torch.empty((n, d), device=dev, dtype=torch.float32)
    ws = _lib.workspace(_lib.OP_MAT5, n, m, d, prec, dev)
    _lib.call(
        "fs_mat5", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d, _lib.ptr(f32), _lib.ptr(g32), _lib.ptr(A32), _lib.ptr(out),
        float(eps), float(cost_scale), prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    return out
