"""Host logic of SamplesLoss that needs no device, against outcomes recorded from the reference
(tests/golden/host_api.json, written by tests/golden/make_golden.py): constructor validation, warnings and
derived attributes; parsing and normalisation of the call forms; the epsilon schedule handed to the gradient."""
import json
import os
import warnings

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from flash_sinkhorn_b200.samples_loss import SamplesLoss, _process_args

with open(os.path.join(GOLDEN_DIR, "host_api.json")) as _fh:
    RECORD = json.load(_fh)


def _arg_case(name):
    g = torch.Generator().manual_seed(5)
    x, y = torch.randn(6, 3, generator=g), torch.randn(4, 3, generator=g)
    a, b = torch.rand(6, generator=g) + 0.1, torch.rand(4, generator=g) + 0.1
    xb, yb = torch.randn(2, 6, 3, generator=g), torch.randn(2, 4, 3, generator=g)
    ab, bb = torch.rand(2, 6, generator=g) + 0.1, torch.rand(2, 4, generator=g) + 0.1
    return {
        "xy": (x, y), "axby": (a, x, b, y), "axby_col": (a[:, None], x, b[:, None], y),
        "batched_xy": (xb, yb), "batched_axby": (ab, xb, bb, yb),
        "batched_axby_col": (ab[..., None], xb, bb[..., None], yb),
        "three_args": (a, x, y), "int_x": (x.long(), y), "not_tensor": (x.tolist(), y),
        "bad_ndim": (x[0], y[0]), "batched_x_flat_y": (xb, y), "batch_mismatch": (xb, yb[:1]),
        "dim_mismatch": (x, y[:, :2]), "bad_a": (a[:5], x, b, y), "bad_b_batched": (ab, xb, bb[:, :3], yb),
    }[name]


def _raises(name):
    return {"ValueError": ValueError, "TypeError": TypeError}[name]


@pytest.mark.parametrize("rec", RECORD["constructor"], ids=lambda r: json.dumps(r["kwargs"], sort_keys=True)[:60])
def test_constructor_outcomes(rec):
    kw = {k: (torch.eye(3) if v == "eye3" else v) for k, v in rec["kwargs"].items()}
    loss_name = kw.pop("loss", "sinkhorn")
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        if "error" in rec:
            with pytest.raises(_raises(rec["error"])):
                SamplesLoss(loss_name, **kw)
            return
        obj = SamplesLoss(loss_name, **kw)
    assert sorted({w.category.__name__ for w in caught}) == rec["warnings"]
    for name, want in rec["attrs"].items():
        have = getattr(obj, name)
        if isinstance(want, dict) and "tensor" in want:
            assert list(have.shape) == want["tensor"], name
        elif isinstance(want, float):
            assert have == pytest.approx(want, rel=1e-12), name
        elif isinstance(want, list):
            assert list(have) == want, name
        else:
            assert have == want, name
    assert obj.process_group is None  # the one attribute added here


@pytest.mark.parametrize("rec", RECORD["process_args"], ids=lambda r: f"{r['case']}-{r['options']['normalize']}")
def test_process_args_outcomes(rec):
    args = _arg_case(rec["case"])
    if "error" in rec:
        with pytest.raises(_raises(rec["error"])):
            _process_args(*args, **rec["options"])
        return
    p = _process_args(*args, **rec["options"])
    assert bool(p.batched) == rec["batched"]
    assert list(p.x.shape) == rec["x_shape"] and list(p.y.shape) == rec["y_shape"]
    assert list(p.a_view_shape) == rec["a_view_shape"] and list(p.b_view_shape) == rec["b_view_shape"]
    np.testing.assert_allclose(p.a.double().numpy(), np.array(rec["a"]), rtol=1e-7, atol=0)
    np.testing.assert_allclose(p.b.double().numpy(), np.array(rec["b"]), rtol=1e-7, atol=0)
    assert p.a.dtype == torch.float32 and p.b.dtype == torch.float32


@pytest.mark.parametrize("rec", RECORD["schedule"], ids=lambda r: json.dumps(r["kwargs"], sort_keys=True)[:60])
def test_epsilon_schedule_for_inputs(rec):
    x = torch.tensor(RECORD["schedule_x"], dtype=torch.float32)
    y = torch.tensor(RECORD["schedule_y"], dtype=torch.float32)
    loss = SamplesLoss("sinkhorn", **rec["kwargs"])
    if "error" in rec:
        with pytest.raises(_raises(rec["error"])):
            loss._eps_list_for_inputs(x, y)
        return
    got = [float(e) for e in loss._eps_list_for_inputs(x, y)]
    assert got == rec["eps_list"]  # float64 host arithmetic: bit-identical


def test_cpu_tensors_are_refused():
    x, y = torch.randn(5, 2), torch.randn(4, 2)
    with pytest.raises(ValueError, match="CUDA"):
        SamplesLoss("sinkhorn")(x, y)


def test_marginal_penalty_precedence():
    """Side-specific values win over the two-sided ones, reach means rho = reach**2, and giving both spellings
    of the same quantity is an error (reference sinkhorn_solvers.py:108-130)."""
    from flash_sinkhorn_b200.kernels._common import dampening, resolve_marginal_penalties as res
    assert res(None, None, None, None, None, None) == (None, None)
    assert res(2.0, None, None, None, None, None) == (2.0, 2.0)
    assert res(None, 3.0, None, None, None, None) == (9.0, 9.0)
    assert res(2.0, None, 5.0, None, None, None) == (5.0, 2.0)
    assert res(2.0, None, None, None, None, 0.5) == (2.0, 0.25)
    assert res(None, 3.0, None, 7.0, 2.0, None) == (4.0, 7.0)
    assert res(None, None, None, None, 1.5, None) == (2.25, None)
    for bad in ((1.0, 1.0, None, None, None, None), (None, None, 1.0, None, 1.0, None),
                (None, None, None, 1.0, None, 1.0)):
        with pytest.raises(ValueError):
            res(*bad)
    assert dampening(0.5, None) == 1.0 and dampening(0.5, 2.0) == pytest.approx(0.8)


def test_epsilon_schedule_argument_checks():
    from flash_sinkhorn_b200.kernels._common import epsilon_schedule
    for bad in ((0.0, 0.1, 0.5), (1.0, 0.0, 0.5), (1.0, 0.1, 1.0), (1.0, 0.1, 0.0)):
        with pytest.raises(ValueError):
            epsilon_schedule(*bad)
    sched = epsilon_schedule(4.0, 0.5, 0.5)
    assert sched[0] == 16.0 and sched[-1] == 0.25 and all(a >= b for a, b in zip(sched, sched[1:]))
