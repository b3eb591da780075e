"""The import paths a user of the reference package relies on exist here under the same names (CPU only:
nothing is called, so the CUDA library is not needed)."""
import importlib
import warnings

import pytest

PKG = "flash_sinkhorn_b200"

TOP_LEVEL = ["SamplesLoss", "CGInfo", "conjugate_gradient", "HvpInfo", "geomloss_to_ott_potentials",
             "hvp_x_sqeuclid", "hvp_x_sqeuclid_from_potentials", "inverse_hvp_x_sqeuclid_from_potentials",
             "ImplicitGradInfo", "implicit_grad_x", "implicit_grad_x_from_potentials", "c_transform_fwd",
             "c_transform_cost", "__version__"]

KERNELS_EAGER = ["epsilon_schedule", "max_diameter", "sinkhorn_flashstyle_alternating",
                 "sinkhorn_flashstyle_symmetric", "apply_plan_vec_flashstyle", "apply_plan_mat_flashstyle",
                 "sinkhorn_geomloss_online_grad_sqeuclid", "c_transform_kernel"]

KERNELS_LAZY = ["log_weights", "apply_lse_kernel_sqeuclid", "apply_transport_from_potentials_sqeuclid",
                "update_potential", "apply_plan_vec_sqeuclid", "apply_plan_mat_sqeuclid", "mat5_sqeuclid",
                "precompute_flashsinkhorn_inputs", "compute_bias_f", "compute_bias_g", "flashsinkhorn_lse",
                "flashsinkhorn_symmetric_step", "shifted_to_standard_potentials", "standard_to_shifted_potentials"]

MODULE_NAMES = {
    "samples_loss": ["SamplesLoss"],
    "cg": ["CGInfo", "conjugate_gradient", "SteihaugCGInfo", "steihaug_cg"],
    "hvp": ["HvpInfo", "geomloss_to_ott_potentials", "hvp_x_sqeuclid", "hvp_x_sqeuclid_from_potentials",
            "inverse_hvp_x_sqeuclid_from_potentials"],
    "implicit_grad": ["ImplicitGradInfo", "implicit_grad_x", "implicit_grad_x_from_potentials"],
    "c_transform": ["c_transform_fwd", "c_transform_cost"],
    "sinkhorn_solvers": ["sinkhorn_flashstyle_alternating", "sinkhorn_flashstyle_symmetric"],
    "kernels._common": ["dampening", "log_weights", "max_diameter", "epsilon_schedule"],
    "kernels.sinkhorn_flashstyle_sqeuclid": [
        "sinkhorn_flashstyle_alternating", "sinkhorn_flashstyle_symmetric", "flashsinkhorn_lse",
        "flashsinkhorn_lse_fused", "flashsinkhorn_symmetric_step", "precompute_flashsinkhorn_inputs",
        "compute_bias_f", "compute_bias_g", "shifted_to_standard_potentials", "standard_to_shifted_potentials"],
    "kernels.apply_flash": ["apply_plan_vec_flashstyle", "apply_plan_mat_flashstyle"],
    "kernels.apply_ott": ["mat5_sqeuclid", "apply_plan_vec_sqeuclid", "apply_plan_mat_sqeuclid"],
    "kernels.sinkhorn_triton_apply_sqeuclid": ["apply_plan_vec_sqeuclid", "apply_plan_mat_sqeuclid", "mat5_sqeuclid",
                                               "apply_plan_mat_flashstyle", "apply_plan_vec_flashstyle"],
    "kernels.sinkhorn_triton_grad_sqeuclid": ["sinkhorn_geomloss_online_grad_sqeuclid"],
    "kernels.c_transform_sqeuclid": ["c_transform_kernel"],
    "kernels.sinkhorn_triton_ott_sqeuclid": ["sinkhorn_potentials_sqeuclid", "apply_lse_kernel_sqeuclid",
                                             "update_potential", "apply_transport_from_potentials_sqeuclid"],
    "kernels.sinkhorn_triton_geomloss_sqeuclid": ["sinkhorn_geomloss_online_potentials_sqeuclid",
                                                  "geomloss_to_ott_potentials", "ott_to_geomloss_potentials",
                                                  "dampening", "epsilon_schedule", "log_weights", "max_diameter"],
}


def test_top_level_and_eager_kernel_names():
    pkg = importlib.import_module(PKG)
    for name in TOP_LEVEL:
        assert hasattr(pkg, name), name
    assert set(TOP_LEVEL) == set(pkg.__all__)
    ker = importlib.import_module(PKG + ".kernels")
    for name in KERNELS_EAGER:
        assert name in ker.__dict__, name
    assert set(KERNELS_EAGER) == set(ker.__all__)


@pytest.mark.parametrize("name", KERNELS_LAZY)
def test_lazy_kernel_names_warn(name):
    ker = importlib.import_module(PKG + ".kernels")
    with pytest.warns(DeprecationWarning, match=name):
        assert callable(getattr(ker, name))
    with pytest.raises(AttributeError):
        getattr(ker, "no_such_kernel")


@pytest.mark.parametrize("module", sorted(MODULE_NAMES))
def test_module_paths(module):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", DeprecationWarning)
        mod = importlib.import_module(f"{PKG}.{module}")
    for name in MODULE_NAMES[module]:
        assert hasattr(mod, name), f"{module}.{name}"


def test_retired_kernel_entry_points_raise():
    mod = importlib.import_module(PKG + ".kernels.sinkhorn_triton_geomloss_sqeuclid")
    with pytest.raises(NotImplementedError):
        mod._geomloss_symmetric_step_sqeuclid()


def _signature_cases():
    import json
    import os

    from conftest import GOLDEN_DIR
    with open(os.path.join(GOLDEN_DIR, "api_signatures.json")) as fh:
        return sorted(json.load(fh).items())


@pytest.mark.parametrize("key,params", _signature_cases(), ids=[k for k, _ in _signature_cases()])
def test_signatures_match_reference(key, params):
    """Every parameter of the reference's callable exists here with the same kind and default, positional
    parameters in the same order; anything added here is optional. A callable that takes ``**kwargs`` may
    absorb keyword-only parameters it forwards untouched."""
    import inspect

    module, name = key.split(":")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", DeprecationWarning)
        obj = getattr(importlib.import_module(f"{PKG}.{module}"), name)
    fn = obj.__init__ if inspect.isclass(obj) else obj
    own = {p.name: p for p in inspect.signature(fn).parameters.values() if p.name != "self"}
    absorbs = any(p.kind is p.VAR_KEYWORD for p in own.values())
    for pname, kind, default in params:
        if pname not in own:
            assert absorbs and kind in ("KEYWORD_ONLY", "VAR_KEYWORD"), f"{key}: parameter {pname} missing"
            continue
        assert own[pname].kind.name == kind, f"{key}: {pname} is {own[pname].kind.name}, reference {kind}"
        have = None if own[pname].default is inspect.Parameter.empty else repr(own[pname].default)
        assert have == default, f"{key}: default of {pname} is {have}, reference {default}"
    positional = [p for p, kind, _ in params if kind == "POSITIONAL_OR_KEYWORD"]
    own_positional = [p.name for p in own.values() if p.kind is p.POSITIONAL_OR_KEYWORD]
    assert own_positional[:len(positional)] == positional, key
    known = {p for p, _, _ in params}
    for pname, p in own.items():
        if pname not in known and p.kind not in (p.VAR_KEYWORD, p.VAR_POSITIONAL):
            assert p.default is not inspect.Parameter.empty, f"{key}: extra parameter {pname} must be optional"
