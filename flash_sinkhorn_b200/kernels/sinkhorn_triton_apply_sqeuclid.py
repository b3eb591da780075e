"""Import-path alias: the reference re-exports the plan applications under this module name."""
from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle  # noqa: F401
from flash_sinkhorn_b200.kernels.apply_ott import mat5_sqeuclid  # noqa: F401
