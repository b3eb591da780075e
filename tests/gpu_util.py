"""Helpers shared by the GPU parity tests (all of which call the CUDA library through the C ABI)."""
import numpy as np
import torch

MODES = ["simt", "fp32", "tf32"]
# Max-relative-error budgets per engine mode against fp64/fp32 references at moderate eps.
TOL = {"simt": 2e-4, "fp32": 2e-4, "tf32": 2e-2}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).cuda()


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def set_mode(monkeypatch, mode):
    monkeypatch.setenv("FLASH_SINKHORN_B200_PREC", mode)


def rel(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))
