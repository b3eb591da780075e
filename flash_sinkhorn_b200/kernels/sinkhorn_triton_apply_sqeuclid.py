"""Import-path alias: the reference re-exports the plan applications under this module name."""
from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle  # noqa: F401
from flash_sinkhorn_b200.kernels.apply_ott import (  # noqa: F401
    apply_plan_mat_sqeuclid,
    apply_plan_vec_sqeuclid,
    mat5_sqeuclid,
)
