"""Analytic (barycentric) gradient of the Sinkhorn cost w.r.t. the point clouds.

``sinkhorn_geomloss_online_grad_sqeuclid`` has the signature of the reference's
``kernels/sinkhorn_triton_grad_sqeuclid.py:891-1207``. One entry point serves every
feature dimension (the reference switches to a separate large-d kernel at :962-1000).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from flash_sinkhorn_b200 import _lib
from flash_sinkhorn_b200.kernels._common import log_weights


def sinkhorn_geomloss_online_grad_sqeuclid(
    x: torch.Tensor,
    y: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    f: torch.Tensor,
    g: torch.Tensor,
    *,
    eps: float,
    allow_tf32: bool = True,
    use_exp2: bool = True,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    block_k: Optional[int] = None,
    num_warps: Optional[int] = None,
    num_stages: int = 2,
    autotune: bool = True,
    grad_scale: Optional[torch.Tensor] = None,
    compute_grad_x: bool = True,
    compute_grad_y: bool = True,
    cost_scale: float = 1.0,
    label_x: Optional[torch.Tensor] = None,
    label_y: Optional[torch.Tensor] = None,
    label_cost_matrix: Optional[torch.Tensor] = None,
    lambda_x: float = 1.0,
    lambda_y: float = 0.0,
    process_group=None,
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``grad_x_i = 2*cs*grad_scale*a_i*(x_i - ybar_i)`` and the symmetric ``grad_y``.

    ``ybar_i`` is the soft-min barycentre ``sum_j w_ij y_j / sum_j w_ij`` with
    ``w_ij = exp((g_j - C_ij)/eps) b_j``. A side that is not requested comes back as None.
    """
    if not x.is_cuda or not y.is_cuda:
        raise ValueError("x and y must be CUDA tensors.")
    if x.ndim != 2 or y.ndim != 2:
        raise ValueError("x and y must be 2D tensors.")
    if a.ndim != 1 or b.ndim != 1:
        raise ValueError("a and b must be 1D tensors.")
    if f.ndim != 1 or g.ndim != 1:
        raise ValueError("f and g must be 1D tensors.")
    n, d = x.shape
    m, d2 = y.shape
    if d != d2:
        raise ValueError("x and y must have the same feature dimension.")
    if a.shape[0] != n or f.shape[0] != n:
        raise ValueError("a and f shapes must match x.")
    if b.shape[0] != m or g.shape[0] != m:
        raise ValueError("b and g shapes must match y.")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError(f"Unsupported dtype for x/y: {x.dtype}")
    if not compute_grad_x and not compute_grad_y:
        return None, None
    dev = _lib.require_cuda(x=x, y=y, a=a, b=b, f=f, g=g)
    # Label-augmented cost lambda_x*cs|x-y|^2 + lambda_y*cs*W[label, label'] inside the weights
    # (reference :225-236); the barycentric formula itself only gains the factor lambda_x (:275).
    labels = _lib.LabelCost.make(label_x, label_y, label_cost_matrix, lambda_x, lambda_y, n, m, dev)
    x32, y32, a32, b32, f32, g32 = map(_lib.f32c, (x, y, a, b, f, g))
    la, lb = log_weights(a32).contiguous(), log_weights(b32).contiguous()
    gs = None
    if grad_scale is not None:
        if grad_scale.numel() != 1:
            raise ValueError("grad_scale must be a scalar tensor.")
        if grad_scale.device != x.device:
            raise ValueError("grad_scale must be on the same device as x.")
        gs = _lib.f32c(grad_scale.detach().reshape(1))
    prec = _lib.precision_id(allow_tf32)
    multi_gpu = process_group is not None and torch.distributed.get_world_size(process_group) > 1
    if labels is not None and multi_gpu:
        raise NotImplementedError("The label cost is not available in the multi-GPU sharded gradient.")
    if multi_gpu:
        from flash_sinkhorn_b200.distributed import grad_sharded  # rows sharded over the ranks, then all-gathered
        return grad_sharded(x32, y32, a32, b32, la, lb, f32, g32, gs, float(eps), float(cost_scale), prec,
                            bool(compute_grad_x), bool(compute_grad_y), process_group)
    gx = torch.empty((n, d), device=dev, dtype=torch.float32) if compute_grad_x else None
    gy = torch.empty((m, d), device=dev, dtype=torch.float32) if compute_grad_y else None
    ws = _lib.workspace(_lib.OP_GRAD, n, m, d, prec, dev, labels.V if labels else 0)
    _lib.call(
        "fs_grad", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d,
        _lib.ptr(a32), _lib.ptr(b32), _lib.ptr(la), _lib.ptr(lb), _lib.ptr(f32), _lib.ptr(g32),
        _lib.ptr(gs), _lib.ptr(gx), _lib.ptr(gy),
        float(eps), float(cost_scale), prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
        labels.ref if labels else None,
    )
    return gx, gy
