"""Host-side scalars and small tensor helpers shared by the solver and kernel wrappers.

Behavioural mirror of the reference's ``kernels/_common.py`` (dampening :20-36,
log_weights :39-44, max_diameter :47-53, epsilon_schedule :56-90). The Triton
autotune helpers of that file have no counterpart here.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

_LOG_ZERO_WEIGHT = -100000.0  # log of a non-positive weight (finite on purpose)


def dampening(eps: float, rho: Optional[float]) -> float:
    """KL-relaxation factor ``1/(1+eps/rho)``; 1 for a hard marginal (``rho is None``)."""
    return 1.0 if rho is None else 1.0 / (1.0 + eps / rho)


def log_weights(w: torch.Tensor) -> torch.Tensor:
    """``log(w)`` in fp32 with non-positive weights mapped to -1e5 (not -inf)."""
    w32 = w.float()
    return torch.where(w32 > 0, w32.log(), torch.full_like(w32, _LOG_ZERO_WEIGHT))


def max_diameter(x: torch.Tensor, y: torch.Tensor) -> float:
    """Diagonal of the joint bounding box of the two clouds (a host float; synchronises)."""
    xf, yf = x.float(), y.float()
    lo = torch.minimum(xf.amin(dim=0), yf.amin(dim=0))
    hi = torch.maximum(xf.amax(dim=0), yf.amax(dim=0))
    return (hi - lo).norm().item()


def epsilon_schedule(diameter: float, blur: float, scaling: float, p: float = 2.0) -> List[float]:
    """GeomLoss annealing schedule: ``diameter**p``, then a geometric descent with ratio
    ``scaling**p`` evaluated in float64 log-space, then ``blur**p``."""
    if diameter <= 0:
        raise ValueError("diameter must be > 0.")
    if blur <= 0:
        raise ValueError("blur must be > 0.")
    if not (0.0 < scaling < 1.0):
        raise ValueError("scaling must be in (0, 1).")
    start, stop, step = p * np.log(diameter), p * np.log(blur), p * np.log(scaling)
    ladder = [float(np.exp(v)) for v in np.arange(start, stop, step)]
    return [diameter**p] + ladder + [blur**p]


def resolve_marginal_penalties(
    rho: Optional[float],
    reach: Optional[float],
    rho_x: Optional[float],
    rho_y: Optional[float],
    reach_x: Optional[float],
    reach_y: Optional[float],
) -> Tuple[Optional[float], Optional[float]]:
    """Collapse the six ways of giving marginal penalties into ``(rho_x, rho_y)``.

    Precedence as in the reference solvers (sinkhorn_solvers.py:108-130, :397-419):
    side-specific rho/reach first, then the two-sided ``rho``, then ``reach`` (rho = reach**2).
    """
    if rho is not None and reach is not None:
        raise ValueError("Specify either rho or reach, not both.")
    if reach is not None:
        rho = reach**2
    if rho is not None:
        if rho_x is None and reach_x is None:
            rho_x = rho
        if rho_y is None and reach_y is None:
            rho_y = rho
    if reach_x is not None:
        if rho_x is not None:
            raise ValueError("Specify either rho_x or reach_x, not both.")
        rho_x = reach_x**2
    if reach_y is not None:
        if rho_y is not None:
            raise ValueError("Specify either rho_y or reach_y, not both.")
        rho_y = reach_y**2
    return rho_x, rho_y


def validate_device(x: torch.Tensor, named: Sequence[Tuple[str, Optional[torch.Tensor]]]) -> None:
    """Every given tensor must live on x's CUDA device (reference :98-118)."""
    for name, t in named:
        if t is None:
            continue
        if not t.is_cuda or t.device != x.device:
            where = t.device if t.is_cuda else "CPU"
            raise ValueError(f"{name} must be on the same CUDA device as x ({x.device}), got {where}")
