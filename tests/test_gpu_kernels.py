"""Single-kernel parity on the GPU: CUDA path (through the C ABI) vs fixtures made by the reference and
vs the CPU oracle, in all three engine modes."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from gpu_util import MODES, TOL, dev, host, rel, set_mode
from oracle import dense_sinkhorn as O

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


@pytest.mark.parametrize("mode", MODES)
def test_kernels_match_reference_fixtures(monkeypatch, mode):
    from flash_sinkhorn_b200.kernels._common import log_weights
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
    from flash_sinkhorn_b200.kernels.apply_ott import mat5_sqeuclid
    from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import (
        flashsinkhorn_lse, flashsinkhorn_lse_fused, flashsinkhorn_symmetric_step)

    set_mode(monkeypatch, mode)
    tol = TOL[mode]
    z = load_golden("kernels_small")
    x, y, a, b, fh, gh = (dev(z[k]) for k in ("x", "y", "a", "b", "f_hat", "g_hat"))
    eps, cs = float(z["eps"]), float(z["cost_scale"])
    la, lb = log_weights(a), log_weights(b)
    assert rel(host(flashsinkhorn_lse(x, y, gh / eps + lb, eps, cost_scale=cs, damping=0.8)), z["lse_raw"]) < tol
    assert rel(host(flashsinkhorn_lse_fused(x, y, gh, lb, eps, cost_scale=cs)), z["lse_fused"]) < tol
    sf, sg = flashsinkhorn_symmetric_step(x, y, fh, gh, la, lb, eps, cost_scale=cs, alpha=0.5,
                                          damping_f=0.9, damping_g=0.7)
    assert rel(host(sf), z["step_f"]) < tol and rel(host(sg), z["step_g"]) < tol
    kw = dict(eps=eps, cost_scale=cs)
    vm, vn, mm, mn, sc = (dev(z[k]) for k in ("vec_m", "vec_n", "mat_m", "mat_n", "scale"))
    ptol = 5 * tol
    assert rel(host(apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, vm, axis=1, **kw)), z["apply_vec_axis1"]) < ptol
    assert rel(host(apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, vn, axis=0, **kw)), z["apply_vec_axis0"]) < ptol
    assert rel(host(apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, mm, axis=1, **kw)), z["apply_mat_axis1"]) < ptol
    assert rel(host(apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, mm, axis=1, scale=sc, **kw)),
               z["apply_mat_axis1_scaled"]) < ptol
    assert rel(host(apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, mn, axis=0, **kw)), z["apply_mat_axis0"]) < ptol
    gx, gy = sinkhorn_geomloss_online_grad_sqeuclid(x, y, a, b, dev(z["f_std"]), dev(z["g_std"]), eps=eps,
                                                    cost_scale=cs, grad_scale=torch.tensor(1.7).cuda())
    assert rel(host(gx), z["grad_x"]) < ptol and rel(host(gy), z["grad_y"]) < ptol
    out = mat5_sqeuclid(x, y, dev(z["f_ott"]), dev(z["g_ott"]), mn, eps=eps, cost_scale=cs)
    assert rel(host(out), z["mat5"]) < ptol


SHAPES = [(1, 1, 1), (1, 7, 3), (7, 1, 1), (31, 33, 3), (64, 64, 8), (65, 127, 16), (129, 100, 24),
          (130, 257, 64), (200, 129, 65), (96, 300, 128), (40, 50, 200)]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("n,m,d", SHAPES)
def test_lse_and_apply_ragged_shapes_vs_oracle(monkeypatch, mode, n, m, d):
    """Ragged / tiny / odd shapes: every row and column must be handled, nothing read out of bounds."""
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse_fused

    set_mode(monkeypatch, mode)
    rng = np.random.default_rng(n * 10007 + m * 101 + d)
    x = (rng.standard_normal((n, d)) / np.sqrt(d)).astype(np.float32)
    y = (0.2 + rng.standard_normal((m, d)) / np.sqrt(d)).astype(np.float32)
    a = rng.random(n).astype(np.float32) + 0.1
    b = rng.random(m).astype(np.float32) + 0.1
    a, b = a / a.sum(), b / b.sum()
    if n > 3:
        a[2] = 0.0  # a zero weight exercises the -1e5 log-weight path
    eps, cs = 0.3, 0.5
    fh = (-cs * (x**2).sum(1) + 0.05 * rng.standard_normal(n)).astype(np.float32)
    gh = (-cs * (y**2).sum(1) + 0.05 * rng.standard_normal(m)).astype(np.float32)
    la, lb = O.log_weights(a), O.log_weights(b)
    X, Y, FH, GH, LA, LB = (a_.astype(np.float64) for a_ in (x, y, fh, gh, la, lb))
    tol = TOL[mode]
    got = flashsinkhorn_lse_fused(dev(x), dev(y), dev(gh), dev(lb), eps, cost_scale=cs, damping=0.9)
    assert rel(host(got), O.lse_update_fused(X, Y, GH, LB, eps, cs, 0.9)) < tol
    got = flashsinkhorn_lse_fused(dev(y), dev(x), dev(fh), dev(la), eps, cost_scale=cs)
    assert rel(host(got), O.lse_update_fused(Y, X, FH, LA, eps, cs)) < tol
    v = rng.standard_normal(m).astype(np.float32)
    V = rng.standard_normal((n, d)).astype(np.float32)
    args = (dev(x), dev(y), dev(fh), dev(gh), dev(la), dev(lb))
    got = apply_plan_vec_flashstyle(*args, dev(v), eps=eps, axis=1, cost_scale=cs)
    assert rel(host(got), O.apply_vec(X, Y, FH, GH, LA, LB, v.astype(np.float64), eps, 1, cs)) < 5 * tol
    got = apply_plan_mat_flashstyle(*args, dev(V), eps=eps, axis=0, cost_scale=cs)
    assert rel(host(got), O.apply_mat(X, Y, FH, GH, LA, LB, V.astype(np.float64), eps, 0, cs)) < 5 * tol


def test_results_are_deterministic():
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse_fused
    g = torch.Generator().manual_seed(5)
    x, y = torch.randn(777, 64, generator=g).cuda(), torch.randn(1030, 64, generator=g).cuda()
    gh = -(y**2).sum(1)
    lb = torch.full((1030,), -np.log(1030.0)).cuda()
    for tf32 in (True, False):
        r1 = flashsinkhorn_lse_fused(x, y, gh, lb, 0.5, allow_tf32=tf32)
        r2 = flashsinkhorn_lse_fused(x, y, gh, lb, 0.5, allow_tf32=tf32)
        assert torch.equal(r1, r2)


def test_single_update_matches_torch_logsumexp():
    """Known-answer check in the style of the reference's test_flashstyle_parity.py:208-276."""
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse
    g = torch.Generator().manual_seed(0)
    n, m, d, eps = 300, 212, 32, 0.1
    x, y = torch.randn(n, d, generator=g).cuda(), torch.randn(m, d, generator=g).cuda()
    bias = torch.randn(m, generator=g).cuda()
    want = -eps * torch.logsumexp((2.0 / eps) * (x.double() @ y.double().T) + bias.double()[None, :], dim=1)
    got = flashsinkhorn_lse(x, y, bias, eps, allow_tf32=False)
    torch.testing.assert_close(got.double(), want, rtol=1e-4, atol=1e-4)
    got_tf32 = flashsinkhorn_lse(x, y, bias, eps, allow_tf32=True)
    torch.testing.assert_close(got_tf32.double(), want, rtol=5e-3, atol=5e-2)


def test_argument_errors():
    from flash_sinkhorn_b200 import SamplesLoss
    from flash_sinkhorn_b200._lib import FlashSinkhornError, call
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse
    x, y = torch.randn(8, 4).cuda(), torch.randn(6, 4).cuda()
    with pytest.raises(ValueError):
        flashsinkhorn_lse(x.cpu(), y, torch.zeros(6).cuda(), 0.1)
    with pytest.raises(ValueError):
        flashsinkhorn_lse(x, y, torch.zeros(5).cuda(), 0.1)
    with pytest.raises(ValueError):
        flashsinkhorn_lse(x, torch.randn(6, 5).cuda(), torch.zeros(6).cuda(), 0.1)
    z8, z6 = torch.zeros(8).cuda(), torch.zeros(6).cuda()
    with pytest.raises(AssertionError):
        apply_plan_vec_flashstyle(x, y, z8, z6, z8, z6, torch.zeros(8).cuda(), eps=0.1, axis=1)
    with pytest.raises(ValueError):
        apply_plan_mat_flashstyle(x, y, z8, z6, z8, z6, torch.zeros(6, 4).cuda(), eps=0.1, axis=2)
    with pytest.raises(ValueError):
        apply_plan_mat_flashstyle(x, y, z8, z6, z8, z6, torch.zeros(8, 4).cuda(), eps=0.1, axis=0, scale=z6)
    with pytest.raises(FlashSinkhornError):  # eps <= 0 is rejected by the C ABI itself
        flashsinkhorn_lse(x, y, z6, 0.0)
    with pytest.raises(TypeError):
        SamplesLoss()(x, y, x)
    with pytest.raises(ValueError):
        SamplesLoss()(x.cpu(), y.cpu())


@pytest.mark.parametrize("n,m", [(130, 40000), (40000, 130), (300, 9000), (5000, 5000), (2600, 777), (257, 1)])
@pytest.mark.parametrize("ctas", [None, 1, 7, 148])
def test_lse_work_split_shapes(monkeypatch, n, m, ctas):
    """The tensor-core LSE pass cuts (row block, column tile) items into one contiguous range per CTA: row
    blocks shared by up to 16 CTAs, CTAs spanning several row blocks, and forced CTA counts must all give the
    torch.logsumexp answer (fp32-exact mode) and run-to-run identical bits."""
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse
    lib = _lib.load()
    previous = lib.fs_set_cta_limit(0 if ctas is None else ctas)
    try:
        _check_lse_work_split(n, m)
    finally:
        lib.fs_set_cta_limit(previous)


def _check_lse_work_split(n, m):
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse
    g = torch.Generator().manual_seed(n + 3 * m)
    d, eps = 16, 0.25
    x = (torch.randn(n, d, generator=g) / 4).cuda()
    y = (torch.randn(m, d, generator=g) / 4).cuda()
    bias = torch.randn(m, generator=g).cuda()
    want = -eps * torch.logsumexp((2.0 / eps) * (x.double() @ y.double().T) + bias.double()[None, :], dim=1)
    got = flashsinkhorn_lse(x, y, bias, eps, allow_tf32=False)
    torch.testing.assert_close(got.double(), want, rtol=1e-4, atol=1e-4)
    assert torch.equal(got, flashsinkhorn_lse(x, y, bias, eps, allow_tf32=False))
    got_tf32 = flashsinkhorn_lse(x, y, bias, eps, allow_tf32=True)
    torch.testing.assert_close(got_tf32.double(), want, rtol=5e-3, atol=5e-2)
    assert _lib.load().fs_device_error() == 0


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["a", "b"])
def test_c_transform_vs_reference(monkeypatch, mode, name):
    """Hard c-transform (values, arg-min, semi-dual objective and Danskin gradients) against the reference's
    results; the exact-product modes must reproduce every index."""
    from flash_sinkhorn_b200 import c_transform_cost, c_transform_fwd
    set_mode(monkeypatch, mode)
    z = load_golden("c_transform_small")
    x, y, psi, wa, wb = (dev(z[name + k]) for k in ("_x", "_y", "_psi", "_wa", "_wb"))
    cs = float(z[name + "_cs"])
    c, idx = c_transform_fwd(x, y, psi, cost_scale=cs, allow_tf32=(mode == "tf32"))
    assert idx.dtype == torch.int64 and not c.requires_grad
    want_c, want_idx = z[name + "_c"], z[name + "_idx"]
    if mode == "tf32":
        # TF32 scores may pick a different near-minimal target; its true cost must be within TF32 noise
        full = O.c_transform(z[name + "_x"].astype(np.float64), z[name + "_y"].astype(np.float64),
                             z[name + "_psi"].astype(np.float64), cs)[0]
        X, Y, P = (z[name + k].astype(np.float64) for k in ("_x", "_y", "_psi"))
        picked = cs * ((X - Y[idx.cpu().numpy()]) ** 2).sum(1) - P[idx.cpu().numpy()]
        assert np.abs(picked - full).max() < 5e-2 and np.abs(host(c) - want_c).max() < 5e-2
        assert (idx.cpu().numpy() == want_idx).mean() > 0.9
        return
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.abs(host(c) - want_c).max() < 1e-4
    xr, pr = x.clone().requires_grad_(True), psi.clone().requires_grad_(True)
    loss = c_transform_cost(xr, y, pr, cost_scale=cs, allow_tf32=False, a=wa, b=wb)
    gx, gp = torch.autograd.grad(loss, [xr, pr])
    assert abs(loss.item() - float(z[name + "_loss"])) < 1e-5 * max(1.0, abs(float(z[name + "_loss"])))
    assert rel(host(gx), z[name + "_grad_x"]) < 1e-5 and np.abs(host(gp) - z[name + "_grad_psi"]).max() < 1e-6
    with pytest.raises(NotImplementedError):
        c_transform_fwd(x, y.clone().requires_grad_(True), psi)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("n,m,d", [(1, 96, 4), (500, 300, 64), (3000, 40000, 16), (40000, 130, 8)])
def test_c_transform_shapes_and_ties(monkeypatch, mode, n, m, d):
    """Tie-break (smallest index among equal minima, also across tiles, column parts and CTAs) and large /
    ragged shapes against torch on the GPU."""
    from flash_sinkhorn_b200 import c_transform_fwd
    set_mode(monkeypatch, mode)
    if (n, m) == (1, 96):
        z = load_golden("c_transform_small")
        _, idx = c_transform_fwd(torch.zeros(1, 4).cuda(), dev(z["tie_y"]), torch.zeros(96).cuda(),
                                 allow_tf32=(mode == "tf32"))
        assert idx.item() == 0
        return
    g = torch.Generator().manual_seed(n + m)
    x = torch.randn(n, d, generator=g).cuda()
    y = torch.randn(m, d, generator=g).cuda()
    y[m // 2:] = y[: m - m // 2]          # every target exists twice: ties everywhere, the first copy must win
    psi = torch.randn(m, generator=g).cuda()
    psi[m // 2:] = psi[: m - m // 2]
    c, idx = c_transform_fwd(x, y, psi, allow_tf32=(mode == "tf32"))
    assert int(idx.max()) < m - m // 2 or m % 2 == 1
    assert int((idx >= (m + 1) // 2).sum()) == 0
    rows = slice(0, min(n, 2000))
    cost = ((x[rows, None, :].double() - y[None, : (m + 1) // 2, :].double()) ** 2).sum(-1) - psi[None, : (m + 1) // 2].double() \
        if m <= 400 else None
    if cost is not None:
        want, widx = cost.min(dim=1)
        tol = 5e-2 if mode == "tf32" else 1e-4
        assert (c[rows].double() - want).abs().max() < tol
        if mode != "tf32":
            assert torch.equal(idx[rows], widx)
    else:
        picked = ((x.double() - y[idx].double()) ** 2).sum(1) - psi[idx].double()
        assert (picked - c.double()).abs().max() < (5e-2 if mode == "tf32" else 2e-4)


@pytest.mark.parametrize("tf32", [True, False])
@pytest.mark.parametrize("n,m,d,vec", [(2100, 4200, 16, False), (4200, 2100, 40, False), (2305, 5000, 8, True),
                                       (300, 9000, 24, False), (1300, 4100, 100, False), (700, 4100, 140, False)])
@pytest.mark.parametrize("split", [0, 1, 2, 3, 4])
def test_plan_times_matrix_work_split(n, m, d, vec, split, tf32):
    """The plan-times-matrix kernel with the row operand resident cuts the column range of a row block into
    shares, one CTA each, that the last CTA to finish adds in share order: every share count (forced through
    the test knob) must give the dense fp64 answer, ragged last row block included, and identical bits from
    run to run."""
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
    lib = _lib.load()
    g = torch.Generator().manual_seed(n + 7 * m + d)
    eps, cs = 0.3, 0.5
    x = (torch.randn(n, d, generator=g) / d ** 0.5).cuda()
    y = (0.2 + torch.randn(m, d, generator=g) / d ** 0.5).cuda()
    fh = -cs * (x ** 2).sum(1) + 0.05 * torch.randn(n, generator=g).cuda()
    gh = -cs * (y ** 2).sum(1) + 0.05 * torch.randn(m, generator=g).cuda()
    la = torch.log_softmax(torch.randn(n, generator=g), 0).cuda()
    lb = torch.log_softmax(torch.randn(m, generator=g), 0).cuda()
    xd, yd = x.double(), y.double()
    logit = (fh.double()[:, None] + gh.double()[None] + 2 * cs * xd @ yd.T) / eps + la.double()[:, None] + lb.double()[None]
    P = torch.exp(logit)
    v = torch.randn(m, generator=g).cuda() if vec else torch.randn(m, d, generator=g).cuda()
    apply = apply_plan_vec_flashstyle if vec else apply_plan_mat_flashstyle
    previous = lib.fs_set_pv_split(split)
    try:
        got = apply(x, y, fh, gh, la, lb, v, eps=eps, axis=1, cost_scale=cs, allow_tf32=tf32)
        again = apply(x, y, fh, gh, la, lb, v, eps=eps, axis=1, cost_scale=cs, allow_tf32=tf32)
    finally:
        lib.fs_set_pv_split(previous)
    want = P @ v.double()
    err = float((got.double() - want).abs().max() / want.abs().max())
    assert err < (2e-2 if tf32 else 2e-4), err
    assert torch.equal(got, again)
    assert lib.fs_device_error() == 0
