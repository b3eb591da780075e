"""flash_sinkhorn_b200: streaming entropic optimal transport on NVIDIA B200 (sm_100a).

Same public surface as the reference package ``flash_sinkhorn`` 0.3.2 for its streaming
Sinkhorn path: ``SamplesLoss``, the analytic gradient and HVP through autograd, the
low-level solvers and plan applications under :mod:`flash_sinkhorn_b200.kernels`.
All device work runs in hand-written CUDA kernels loaded from
``lib/libflashsinkhorn_b200.so`` through a C ABI (``include/flash_sinkhorn_b200.h``).
"""
from flash_sinkhorn_b200.samples_loss import SamplesLoss
from flash_sinkhorn_b200.cg import CGInfo, conjugate_gradient
from flash_sinkhorn_b200.hvp import (
    HvpInfo,
    geomloss_to_ott_potentials,
    hvp_x_sqeuclid,
    hvp_x_sqeuclid_from_potentials,
    inverse_hvp_x_sqeuclid_from_potentials,
)
from flash_sinkhorn_b200.c_transform import c_transform_cost, c_transform_fwd
from flash_sinkhorn_b200.implicit_grad import ImplicitGradInfo, implicit_grad_x, implicit_grad_x_from_potentials

__all__ = [
    "SamplesLoss",
    "CGInfo",
    "conjugate_gradient",
    "HvpInfo",
    "geomloss_to_ott_potentials",
    "hvp_x_sqeuclid",
    "hvp_x_sqeuclid_from_potentials",
    "inverse_hvp_x_sqeuclid_from_potentials",
    "ImplicitGradInfo",
    "implicit_grad_x",
    "implicit_grad_x_from_potentials",
    "c_transform_fwd",
    "c_transform_cost",
    "__version__",
]
__version__ = "0.1.0"
