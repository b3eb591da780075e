"""Multi-threaded dense CPU baseline (PyTorch fp32) for the timed ``cpu_baseline`` legs.  TEST/BENCH ONLY.

The same dense log-domain symmetric Sinkhorn the reference ships as its CPU-runnable path
(testing/reference_sinkhorn.py:119-192: full cost matrix, ``torch.logsumexp`` soft-mins,
Jacobi averaging), restated so it can run row-chunked: at n = m = 50,000 the cost matrix
is 10 GB, so each soft-min is evaluated over blocks of rows / columns with identical
arithmetic per entry. Never imported by the product.
"""
from __future__ import annotations

import time
from typing import Tuple

import torch


def _softmin_rows(x, y, y2, pot, logw, eps, cost_scale, chunk):
    """-eps * LSE_j[(pot_j - C_ij)/eps + logw_j] for every row i, in row blocks of `chunk`."""
    out = torch.empty(x.shape[0], dtype=torch.float32)
    for s in range(0, x.shape[0], chunk):
        xs = x[s:s + chunk]
        cost = cost_scale * ((xs * xs).sum(1, keepdim=True) + y2[None, :] - 2.0 * xs @ y.t())
        out[s:s + chunk] = -eps * torch.logsumexp((pot[None, :] - cost) / eps + logw[None, :], dim=1)
    return out


def symmetric_steps(x, y, a, b, eps: float, n_steps: int, cost_scale: float = 1.0, chunk: int = 4096
                    ) -> Tuple[torch.Tensor, torch.Tensor, float, int]:
    """Init step + `n_steps` averaged Jacobi steps at fixed eps. Returns (f, g, seconds, entries)."""
    x, y = x.float(), y.float()
    x2, y2 = (x * x).sum(1), (y * y).sum(1)
    la, lb = a.float().log(), b.float().log()
    n, m = x.shape[0], y.shape[0]
    t0 = time.perf_counter()
    f = _softmin_rows(x, y, y2, torch.zeros(m), lb, eps, cost_scale, chunk)
    g = _softmin_rows(y, x, x2, torch.zeros(n), la, eps, cost_scale, chunk)
    for _ in range(n_steps):
        ft = _softmin_rows(x, y, y2, g, lb, eps, cost_scale, chunk)
        gt = _softmin_rows(y, x, x2, f, la, eps, cost_scale, chunk)
        f, g = 0.5 * (f + ft), 0.5 * (g + gt)
    dt = time.perf_counter() - t0
    return f, g, dt, 2 * n * m * (n_steps + 1)
