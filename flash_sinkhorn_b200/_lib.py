"""ctypes binding of ``libflashsinkhorn_b200.so`` (the sm_100a CUDA engine).

The shared library is the product; this module only marshals PyTorch device
pointers, the current CUDA stream and a caller-owned workspace into the C ABI
declared in ``include/flash_sinkhorn_b200.h``. There is no fallback: if the
library is missing, or a call returns a non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_size_t, c_void_p
from typing import Optional

import torch

_LIB_NAME = "libflashsinkhorn_b200.so"
_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", _LIB_NAME)

PREC_TF32 = 0
PREC_FP32 = 1
PREC_SIMT = 2

OP_LSE = 0
OP_STEP = 1
OP_SOLVE_SYMMETRIC = 2
OP_SOLVE_ALTERNATING = 3
OP_APPLY_VEC = 4
OP_APPLY_MAT = 5
OP_GRAD = 6
OP_MAT5 = 7
OP_SCHUR = 8

_STATUS_NAMES = {
    1: "FS_ERR_BAD_ARG",
    2: "FS_ERR_UNSUPPORTED",
    3: "FS_ERR_CUDA",
    4: "FS_ERR_TIMEOUT",
    5: "FS_ERR_WORKSPACE",
}

# name -> (restype, argtypes); mirrors include/flash_sinkhorn_b200.h one to one.
_P = c_void_p
SIGNATURES = {
    "fs_version": (c_int, []),
    "fs_last_error": (c_char_p, []),
    "fs_device_arch": (c_int, []),
    "fs_launch_count": (ctypes.c_longlong, []),
    "fs_device_error": (c_int, []),
    "fs_clear_device_error": (c_int, []),
    "fs_apply_mat_plan_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "fs_micro_exp_rate": (c_double, [c_int, c_int]),
    "fs_micro_mma_cycles": (c_double, [c_int, c_int]),
    "fs_set_reserved_sms": (c_int, [c_int]),
    "fs_set_cta_limit": (c_int, [c_int]),
    "fs_set_wide_tile_min_chunks": (c_int, [c_int]),
    "fs_set_prefer_streamed": (c_int, [c_int]),
    "fs_set_pv_split": (c_int, [c_int]),
    "fs_engine": (c_int, [c_int, c_int, c_int, c_int]),
    "fs_plan_ctas": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "fs_plan_pv_split": (c_int, [c_int, c_int, c_int, c_int, ctypes.POINTER(c_int)]),
    "fs_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "fs_workspace_bytes_labels": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "fs_lse": (c_int, [_P, _P, c_int, c_int, c_int, _P, _P, _P, c_float, c_float, c_float, c_int, _P, c_size_t, _P]),
    "fs_c_transform": (c_int, [_P, _P, c_int, c_int, c_int, _P, c_float, _P, _P, c_int, _P, c_size_t, _P]),
    "fs_symmetric_step": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P,
         c_float, c_float, c_float, c_float, c_float, c_int, _P, c_size_t, _P, _P],
    ),
    "fs_symmetric_step_range": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P,
         c_float, c_float, c_float, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P],
    ),
    "fs_symmetric_step_range_tiles": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P,
         c_float, c_float, c_float, c_float, c_float, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P,
         c_int, _P, c_size_t, _P],
    ),
    "fs_symmetric_step_multi": (c_int, [_P, c_int, c_int, c_int, _P]),
    "fs_solve_symmetric_batched": (c_int, [_P, c_int, c_int, c_int, c_float, c_double, c_double, c_int, _P]),
    "fs_grad_range": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_float, c_float,
         c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P],
    ),
    "fs_solve_symmetric": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, c_int, c_int, c_float, c_double, c_double,
         c_double, c_int, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_size_t, _P, _P],
    ),
    "fs_solve_alternating": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, c_int, c_int, c_float, c_double, c_double,
         c_int, c_double, c_int, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_size_t, _P],
    ),
    "fs_apply_vec": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, c_float, c_int, c_float, c_int, _P, c_size_t, _P],
    ),
    "fs_apply_mat": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int, _P, _P, c_float, c_int, c_float,
         c_int, _P, c_size_t, _P],
    ),
    "fs_apply_mat_static": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int, _P, _P, c_float, c_int, c_float, _P],
    ),
    "fs_grad": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_float, c_float,
         c_int, _P, c_size_t, _P, _P],
    ),
    "fs_mat5": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, c_float, c_float, c_int, _P, c_size_t, _P],
    ),
    "fs_plan_session_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "fs_plan_session_begin": (
        c_int, [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, c_float, c_float, c_int, _P, c_size_t, _P]),
    "fs_plan_session_apply": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, c_int, _P, c_float, _P, c_int, c_float, c_float,
         c_int, _P, c_size_t, _P]),
    "fs_plan_session_cg": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_float, c_float, c_int,
         c_float, c_float, c_int, _P, c_size_t, _P]),
    "fs_schur_cg": (
        c_int,
        [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_float, c_float, c_int,
         c_float, c_float, c_int, _P, c_size_t, _P],
    ),
}

_lib: Optional[ctypes.CDLL] = None


class FlashSinkhornError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def library_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the CUDA library (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_NAME} not found at {_LIB_PATH}. Build it with "
            "`python -m flash_sinkhorn_b200.build_ext` (needs nvcc with sm_100a support). "
            "There is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(_LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def precision_id(allow_tf32: bool) -> int:
    """``allow_tf32`` of the reference API -> engine precision mode.

    The environment variable FLASH_SINKHORN_B200_PREC (tf32|fp32|simt) overrides it,
    which the tests use to cross-check the engines against each other.
    """
    env = os.environ.get("FLASH_SINKHORN_B200_PREC", "").lower()
    if env == "simt":
        return PREC_SIMT
    if env == "fp32":
        return PREC_FP32
    if env == "tf32":
        return PREC_TF32
    return PREC_TF32 if allow_tf32 else PREC_FP32


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr()


def f32c(t: torch.Tensor) -> torch.Tensor:
    """Contiguous fp32 view/copy (the engine reads fp32 only)."""
    if t.dtype != torch.float32:
        t = t.float()
    return t.contiguous()


def require_cuda(**tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor.")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"{name} must be on the same CUDA device as the other tensors ({dev}), got {t.device}")
    assert dev is not None
    return dev


def workspace(op: int, n: int, m: int, d: int, prec: int, device: torch.device, n_classes: int = 0) -> torch.Tensor:
    """Scratch tensor for one call of ``op``; ``n_classes`` = V of the label cost the call will pass (0 = none)."""
    nbytes = int(load().fs_workspace_bytes_labels(op, n, m, d, prec, int(n_classes)))
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)


class LabelCostStruct(ctypes.Structure):
    """``fs_label_cost`` of the C header."""

    _fields_ = [("label_x", c_void_p), ("label_y", c_void_p), ("W", c_void_p), ("V", c_int),
                ("lambda_x", c_float), ("lambda_y", c_float)]


class LabelCost:
    """Validated label-cost arguments (reference kernels/sinkhorn_flashstyle_sqeuclid.py:1183-1213): int32
    labels on the device of x, a square fp32 table, and the ctypes descriptor that points at them.
    ``LabelCost.make`` returns None when the label cost is inactive (any of the four inputs missing, or
    ``lambda_y == 0``), exactly the reference's ``use_label_cost`` condition."""

    def __init__(self, label_x, label_y, table, lambda_x, lambda_y):
        self.label_x, self.label_y, self.table = label_x, label_y, table
        self.V = int(table.shape[0])
        self.struct = LabelCostStruct(label_x.data_ptr(), label_y.data_ptr(), table.data_ptr(), self.V,
                                      float(lambda_x), float(lambda_y))

    @property
    def ref(self):
        return ctypes.cast(ctypes.pointer(self.struct), c_void_p)

    @staticmethod
    def make(label_x, label_y, label_cost_matrix, lambda_x, lambda_y, n, m, device):
        if label_x is None or label_y is None or label_cost_matrix is None or float(lambda_y) == 0.0:
            return None
        if label_x.shape[0] != n:
            raise ValueError(f"label_x must have length n={n}, got {label_x.shape[0]}")
        if label_y.shape[0] != m:
            raise ValueError(f"label_y must have length m={m}, got {label_y.shape[0]}")
        if label_cost_matrix.ndim != 2:
            raise ValueError("label_cost_matrix must be 2D (V, V)")
        if label_cost_matrix.shape[0] != label_cost_matrix.shape[1]:
            raise ValueError("label_cost_matrix must be square (V, V)")
        V = label_cost_matrix.shape[0]
        for name, lab in (("label_x", label_x), ("label_y", label_y)):
            lo, hi = int(lab.min()), int(lab.max())
            if hi >= V or lo < 0:
                raise ValueError(f"{name} values must be in [0, {V}), got range [{lo}, {hi}]")
        if not float(lambda_x) > 0.0:
            raise ValueError("lambda_x must be > 0 when a label cost is used")
        return LabelCost(label_x.to(dtype=torch.int32, device=device).contiguous(),
                         label_y.to(dtype=torch.int32, device=device).contiguous(),
                         label_cost_matrix.to(dtype=torch.float32, device=device).contiguous(),
                         lambda_x, lambda_y)


class StepItem(ctypes.Structure):
    """``fs_step_item`` of the C header (one row-sharded Jacobi step of one problem)."""

    _fields_ = [("x", c_void_p), ("y", c_void_p), ("n", c_int), ("m", c_int),
                ("f_hat", c_void_p), ("g_hat", c_void_p), ("log_a", c_void_p), ("log_b", c_void_p),
                ("f_out", c_void_p), ("g_out", c_void_p), ("alpha_x", c_void_p), ("beta_y", c_void_p),
                ("eps", c_float), ("w", c_float), ("damp_f", c_float), ("damp_g", c_float), ("cost_scale", c_float),
                ("f_begin", c_int), ("f_end", c_int), ("g_begin", c_int), ("g_end", c_int), ("restage", c_int),
                ("ws", c_void_p), ("ws_bytes", c_size_t),
                ("f_shard", c_int), ("g_shard", c_int), ("pack_stride", c_int)]


class BatchItem(ctypes.Structure):
    """``fs_batch_item`` of the C header (one problem of a batched symmetric solve)."""

    _fields_ = [("x", c_void_p), ("y", c_void_p), ("n", c_int), ("m", c_int), ("log_a", c_void_p), ("log_b", c_void_p),
                ("eps_list_host", c_void_p), ("n_eps", c_int), ("f", c_void_p), ("g", c_void_p),
                ("f_pre", c_void_p), ("g_pre", c_void_p), ("ws", c_void_p), ("ws_bytes", c_size_t)]


def stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def raise_if_device_timeout(device: torch.device) -> None:
    """Raise ``FlashSinkhornError`` (FS_ERR_TIMEOUT) if a kernel of the library gave up one of its bounded waits.

    Meant for the places where the host synchronises anyway (reading an iteration count or a CG record): the
    outputs of the call that timed out are invalid, and its workspace has to be staged again. The word stays set
    until ``fs_clear_device_error``."""
    lib = load()
    with torch.cuda.device(device):
        flag = lib.fs_device_error()
    if flag > 0:
        raise FlashSinkhornError(
            "FS_ERR_TIMEOUT: a streaming kernel gave up a bounded wait; the results of that call are invalid. "
            "Re-stage its workspace (run the call again) and reset the word with fs_clear_device_error().")


def call(name: str, device: torch.device, *args) -> None:
    """Invoke a compute entry point with `device` current; raise on failure."""
    lib = load()
    with torch.cuda.device(device):
        status = getattr(lib, name)(*args)
    if status != 0:
        msg = lib.fs_last_error().decode("utf-8", "replace")
        raise FlashSinkhornError(f"{name} failed with {_STATUS_NAMES.get(status, status)}: {msg}")
