"""HVP term ``Mat5`` with OTT-convention potentials.

``mat5_sqeuclid`` has the signature of the reference's ``kernels/apply_ott.py:453-566``:
``out_i = (-4*cost_scale/eps) * sum_j P_ij (A_i . y_j) y_j`` with
``P_ij = exp((f_i + g_j - C_ij)/eps)``. The reference's deprecated OTT-convention
``apply_plan_*_sqeuclid`` wrappers are not provided.
"""
from __future__ import annotations

from typing import Optional

import torch

from flash_sinkhorn_b200 import _lib
from flash_sinkhorn_b200.kernels._common import validate_device


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
