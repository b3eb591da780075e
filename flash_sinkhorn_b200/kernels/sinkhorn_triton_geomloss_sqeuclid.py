"""Deprecated GeomLoss-convention solver name, kept so that old imports keep working.

Mirrors the reference's ``kernels/sinkhorn_triton_geomloss_sqeuclid.py``:
``sinkhorn_geomloss_online_potentials_sqeuclid`` (:79-235) forwards to
:func:`sinkhorn_flashstyle_symmetric`; the potential-convention converters (:33-76) and the host
scalars of ``_common`` are re-exported; the old kernel entry points (:278-289) raise.
"""
from __future__ import annotations

import warnings

from flash_sinkhorn_b200.hvp import geomloss_to_ott_potentials, ott_to_geomloss_potentials
from flash_sinkhorn_b200.kernels._common import dampening, epsilon_schedule, log_weights, max_diameter
from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric

__all__ = [
    "sinkhorn_geomloss_online_potentials_sqeuclid",
    "geomloss_to_ott_potentials",
    "ott_to_geomloss_potentials",
    "dampening",
    "epsilon_schedule",
    "log_weights",
    "max_diameter",
]

_TILE_KEYS = ("block_m", "block_n", "block_k", "num_warps")


def sinkhorn_geomloss_online_potentials_sqeuclid(x, y, a, b, *, f_init=None, g_init=None, num_stages: int = 2,
                                                 **options):
    """Deprecated alias of :func:`sinkhorn_flashstyle_symmetric` (same keywords, same return tuple).

    As in the reference, warm-start potentials and manual tile sizes are dropped with a ``UserWarning``.
    """
    warnings.warn(
        "sinkhorn_geomloss_online_potentials_sqeuclid is deprecated; use sinkhorn_flashstyle_symmetric "
        "(flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid).",
        DeprecationWarning, stacklevel=2,
    )
    if f_init is not None or g_init is not None:
        warnings.warn("f_init and g_init are ignored here: the solve starts from zero potentials.",
                      UserWarning, stacklevel=2)
    if any(options.get(k) is not None for k in _TILE_KEYS):
        warnings.warn("Manual block sizes (block_m, block_n, block_k, num_warps) are ignored.",
                      UserWarning, stacklevel=2)
    for k in _TILE_KEYS:
        options.pop(k, None)
    return sinkhorn_flashstyle_symmetric(x, y, a, b, **options)


def _geomloss_symmetric_step_sqeuclid_impl(*args, **kwargs):
    raise NotImplementedError(
        "_geomloss_symmetric_step_sqeuclid_impl is deprecated. Use sinkhorn_flashstyle_symmetric instead."
    )


_geomloss_symmetric_step_sqeuclid = _geomloss_symmetric_step_sqeuclid_impl
_geomloss_symmetric_step_sqeuclid_autotune = _geomloss_symmetric_step_sqeuclid_impl
_geomloss_symmetric_step_sqeuclid_autotune_label = _geomloss_symmetric_step_sqeuclid_impl
