"""Kernel launchers. Eager exports match the reference's ``kernels/__init__.py:17-58``;
the names it serves lazily with a DeprecationWarning (:65-97) are served the same way."""
from flash_sinkhorn_b200.kernels._common import epsilon_schedule, max_diameter
from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import (
    sinkhorn_flashstyle_alternating,
    sinkhorn_flashstyle_symmetric,
)
from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid
from flash_sinkhorn_b200.kernels.c_transform_sqeuclid import c_transform_kernel

__all__ = [
    "epsilon_schedule",
    "max_diameter",
    "sinkhorn_flashstyle_alternating",
    "sinkhorn_flashstyle_symmetric",
    "apply_plan_vec_flashstyle",
    "apply_plan_mat_flashstyle",
    "sinkhorn_geomloss_online_grad_sqeuclid",
    "c_transform_kernel",
]

_LAZY = {
    "log_weights": "flash_sinkhorn_b200.kernels._common",
    "apply_lse_kernel_sqeuclid": "flash_sinkhorn_b200.kernels.sinkhorn_triton_ott_sqeuclid",
    "apply_transport_from_potentials_sqeuclid": "flash_sinkhorn_b200.kernels.sinkhorn_triton_ott_sqeuclid",
    "update_potential": "flash_sinkhorn_b200.kernels.sinkhorn_triton_ott_sqeuclid",
    "apply_plan_vec_sqeuclid": "flash_sinkhorn_b200.kernels.apply_ott",
    "apply_plan_mat_sqeuclid": "flash_sinkhorn_b200.kernels.apply_ott",
    "mat5_sqeuclid": "flash_sinkhorn_b200.kernels.apply_ott",
    "precompute_flashsinkhorn_inputs": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
    "compute_bias_f": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
    "compute_bias_g": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
    "flashsinkhorn_lse": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
    "flashsinkhorn_lse_fused": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
    "flashsinkhorn_symmetric_step": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
    "shifted_to_standard_potentials": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
    "standard_to_shifted_potentials": "flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid",
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        import warnings

        warnings.warn(
            f"Importing {name} from flash_sinkhorn_b200.kernels is deprecated. Import from {_LAZY[name]} directly.",
            DeprecationWarning, stacklevel=2,
        )
        return getattr(importlib.import_module(_LAZY[name]), name)
    raise AttributeError(f"module 'flash_sinkhorn_b200.kernels' has no attribute {name!r}")
