"""Streaming plan applications ``P v``, ``P^T v``, ``P V``, ``P^T V`` from shifted potentials.

Call signatures and validation follow the reference's ``kernels/apply_flash.py``
(apply_plan_mat_flashstyle :360-579, apply_plan_vec_flashstyle :835-951), with
``P_ij = a_i b_j exp((f_hat_i + g_hat_j + 2*cost_scale*x_i.y_j)/eps)``.
Triton tuning keywords are accepted and ignored.
"""
from __future__ import annotations

from typing import Optional

import torch

from flash_sinkhorn_b200 import _lib
from flash_sinkhorn_b200.kernels._common import validate_device


def apply_plan_vec_flashstyle(
    x: torch.Tensor,
    y: torch.Tensor,
    f_hat: torch.Tensor,
    g_hat: torch.Tensor,
    log_a: torch.Tensor,
    log_b: torch.Tensor,
    vec: torch.Tensor,
    *,
    eps: float,
    axis: int,
    cost_scale: float = 1.0,
    allow_tf32: bool = False,
    use_exp2: bool = True,
    block_m: int = 64,
    block_n: int = 64,
    block_k: int = 64,
    num_warps: int = 4,
    num_stages: int = 2,
) -> torch.Tensor:
    """``P @ vec`` (``axis=1``, vec of length m) or ``P.T @ vec`` (``axis=0``, length n)."""
    n, d = x.shape
    m = y.shape[0]
    assert f_hat.shape == (n,), f"f_hat shape {f_hat.shape} != ({n},)"
    assert g_hat.shape == (m,), f"g_hat shape {g_hat.shape} != ({m},)"
    assert log_a.shape == (n,), f"log_a shape {log_a.shape} != ({n},)"
    assert log_b.shape == (m,), f"log_b shape {log_b.shape} != ({m},)"
    if axis == 1:
        assert vec.shape == (m,), f"vec shape {vec.shape} != ({m},) for axis=1"
    else:
        assert vec.shape == (n,), f"vec shape {vec.shape} != ({n},) for axis=0"
    dev = _lib.require_cuda(x=x, y=y, f_hat=f_hat, g_hat=g_hat, log_a=log_a, log_b=log_b, vec=vec)
    x32, y32 = _lib.f32c(x), _lib.f32c(y)
    fh, gh, la, lb, v = map(_lib.f32c, (f_hat, g_hat, log_a, log_b, vec))
    prec = _lib.precision_id(allow_tf32)
    out = torch.empty((n if axis == 1 else m,), device=dev, dtype=torch.float32)
    ws = _lib.workspace(_lib.OP_APPLY_VEC, n, m, d, prec, dev)
    _lib.call(
        "fs_apply_vec", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d,
        _lib.ptr(fh), _lib.ptr(gh), _lib.ptr(la), _lib.ptr(lb), _lib.ptr(v), _lib.ptr(out),
        float(eps), 1 if axis == 1 else 0, float(cost_scale),
        prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    return out


def apply_plan_mat_flashstyle(
    x: torch.Tensor,
    y: torch.Tensor,
    f_hat: torch.Tensor,
    g_hat: torch.Tensor,
    log_a: torch.Tensor,
    log_b: torch.Tensor,
    mat: torch.Tensor,
    *,
    eps: float,
    axis: int,
    cost_scale: float = 1.0,
    scale: Optional[torch.Tensor] = None,
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
    """``P @ mat`` (``axis=1``; optional per-row ``scale`` of mat) or ``P.T @ mat`` (``axis=0``)."""
    if axis not in (0, 1):
        raise ValueError("axis must be 0 or 1.")
    if not x.is_cuda:
        raise ValueError("CUDA required.")
    if x.ndim != 2 or y.ndim != 2 or mat.ndim != 2:
        raise ValueError("x, y, mat must be 2D tensors.")
    if f_hat.ndim != 1 or g_hat.ndim != 1:
        raise ValueError("f_hat and g_hat must be 1D.")
    if log_a.ndim != 1 or log_b.ndim != 1:
        raise ValueError("log_a and log_b must be 1D.")
    validate_device(x, [("y", y), ("f_hat", f_hat), ("g_hat", g_hat), ("log_a", log_a),
                        ("log_b", log_b), ("mat", mat), ("scale", scale)])
    n, d = x.shape
    m, d2 = y.shape
    if d != d2:
        raise ValueError("x and y must have the same feature dimension.")
    if f_hat.shape[0] != n or log_a.shape[0] != n:
        raise ValueError("f_hat and log_a must have shape (n,).")
    if g_hat.shape[0] != m or log_b.shape[0] != m:
        raise ValueError("g_hat and log_b must have shape (m,).")
    if axis == 1 and mat.shape != (m, d):
        raise ValueError("For axis=1, mat must have shape (m, d).")
    if axis == 0 and mat.shape != (n, d):
        raise ValueError("For axis=0, mat must have shape (n, d).")
    if scale is not None:
        if axis != 1:
            raise ValueError("scale is only supported for axis=1.")
        if scale.shape != (m,):
            raise ValueError("scale must have shape (m,).")
    dev = x.device
    x32, y32 = _lib.f32c(x), _lib.f32c(y)
    fh, gh, la, lb, v = map(_lib.f32c, (f_hat, g_hat, log_a, log_b, mat))
    sc = None if scale is None else _lib.f32c(scale)
    prec = _lib.precision_id(allow_tf32)
    dv = v.shape[1]
    out = torch.empty((n if axis == 1 else m, dv), device=dev, dtype=torch.float32)
    ws = _lib.workspace(_lib.OP_APPLY_MAT, n, m, d, prec, dev)
    _lib.call(
        "fs_apply_mat", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d,
        _lib.ptr(fh), _lib.ptr(gh), _lib.ptr(la), _lib.ptr(lb),
        _lib.ptr(v), dv, _lib.ptr(sc), _lib.ptr(out),
        float(eps), axis, float(cost_scale),
        prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    return out
