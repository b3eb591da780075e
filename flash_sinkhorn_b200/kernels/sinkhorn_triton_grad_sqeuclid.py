"""Import-path alias: the reference exposes the gradient launcher under this module name."""
from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid  # noqa: F401
