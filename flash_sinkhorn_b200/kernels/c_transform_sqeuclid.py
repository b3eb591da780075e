"""Hard c-transform kernel wrapper: streaming min + arg-min over the factored squared-Euclidean cost.

Signature and semantics of the reference's ``kernels/c_transform_sqeuclid.py:219-354``
(``c_transform_kernel``): for every source point

    min_val_i = min_j [ -2*cost_scale * x_i.y_j + bias_j ],   argmin_i = the smallest such j

with ``bias_j = cost_scale*|y_j|^2 - psi_j``; the caller adds ``cost_scale*|x_i|^2``. The pass runs on the
same staged operands and tile engine as the soft-min update (``fs_c_transform``): TF32 score tiles from
``tcgen05`` with the bias folded into the contraction, a running (max, column) pair per row in registers,
no exponentials. ``block_*``, ``num_warps``, ``num_stages`` and ``autotune`` are accepted and ignored.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from flash_sinkhorn_b200 import _lib

__all__ = ["c_transform_kernel"]


def c_transform_kernel(
    x: torch.Tensor,
    y: torch.Tensor,
    bias: torch.Tensor,
    *,
    cost_scale: float = 1.0,
    allow_tf32: bool = True,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: Optional[int] = None,
    num_stages: int = 3,
    autotune: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(min_vals [n] float32, argmin_idx [n] int64)``."""
    if not x.is_cuda or not y.is_cuda:
        raise ValueError("x and y must be CUDA tensors")
    if x.ndim != 2 or y.ndim != 2:
        raise ValueError("x and y must be 2D tensors")
    if bias.ndim != 1:
        raise ValueError("bias must be 1D tensor")
    n, d = x.shape
    m, d2 = y.shape
    if d != d2:
        raise ValueError("x and y must have same feature dimension")
    if bias.shape[0] != m:
        raise ValueError(f"bias must have length {m}, got {bias.shape[0]}")
    if m == 0:
        raise ValueError("m must be > 0")
    dev = _lib.require_cuda(x=x, y=y, bias=bias)
    x32, y32, b32 = _lib.f32c(x), _lib.f32c(y), _lib.f32c(bias)
    prec = _lib.precision_id(allow_tf32)
    out_val = torch.empty((n,), device=dev, dtype=torch.float32)
    out_idx = torch.empty((n,), device=dev, dtype=torch.int32)
    if n == 0:
        return out_val, out_idx.to(torch.long)
    ws = _lib.workspace(_lib.OP_LSE, n, m, d, prec, dev)
    _lib.call(
        "fs_c_transform", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d, _lib.ptr(b32), float(cost_scale),
        _lib.ptr(out_val), _lib.ptr(out_idx), prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    return out_val, out_idx.to(torch.long)
