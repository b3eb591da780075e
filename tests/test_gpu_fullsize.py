"""Size-independent properties at the full sizes of benchmark configurations 3-5 (the dense oracle cannot run there)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def test_config5_shape_large_d_semi_unbalanced_gradient():
    """n = m = 16384, d = 2048, unit-sphere rows, reach_x = 1, half cost: loss finite and positive, and the
    analytic gradient (any-d entry point) matches a central finite difference of the loss along a random
    direction (the property the reference's large-d tests rely on, test_geomloss_sinkhorn_triton.py:255-322)."""
    from flash_sinkhorn_b200 import SamplesLoss
    gen = torch.Generator().manual_seed(4)
    n = m = 16384
    d = 2048
    x = torch.nn.functional.normalize(torch.randn(n, d, generator=gen), dim=1).cuda()
    y = torch.nn.functional.normalize(torch.randn(m, d, generator=gen), dim=1).cuda()
    loss = SamplesLoss("sinkhorn", blur=0.05, reach_x=1.0, reach_y=None, half_cost=True, use_epsilon_scaling=False,
                       eps=0.0025, n_iters=4, allow_tf32=False)
    xs = x.clone().requires_grad_(True)
    val = loss(xs, y)
    (gx,) = torch.autograd.grad(val, xs)
    assert torch.isfinite(val) and val.item() > 0
    assert torch.isfinite(gx).all() and gx.shape == (n, d)
    # rows of the gradient point from the soft-min barycentre to x_i, scaled by a_i = 1/n
    assert gx.norm(dim=1).max().item() < 4.0 / n
    # directional derivative along the (normalised) gradient itself, by central differences of the loss
    u = gx / gx.norm()
    h = 0.5
    with torch.no_grad():
        fd = (loss(x + h * u, y).item() - loss(x - h * u, y).item()) / (2 * h)
    an = (gx * u).sum().item()
    assert an > 0
    # the envelope gradient at non-converged potentials is approximate; 15 % is the property's bar
    assert abs(fd - an) <= 0.15 * abs(an)


def test_config4_shape_unbalanced_early_stop_counter_and_masses():
    """n = 100000, m = 80000, d = 128, masses 1.0 / 1.3, reach = 1: the device-side early stop fires, the
    iteration counter is consistent, and the relaxed plan's total mass lies between the two input masses."""
    from flash_sinkhorn_b200.kernels._common import log_weights
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
    gen = torch.Generator().manual_seed(3)
    n, m, d = 100000, 80000, 128
    x = torch.randn(n, d, generator=gen).cuda()
    y = (1.5 * torch.randn(m, d, generator=gen)).cuda()
    a = torch.softmax(torch.randn(n, generator=gen), 0).cuda()
    b = (1.3 * torch.softmax(torch.randn(m, generator=gen), 0)).cuda()
    eps = 0.04
    f, g, k = sinkhorn_flashstyle_symmetric(x, y, a, b, use_epsilon_scaling=False, eps=eps, n_iters=60, reach=1.0,
                                            threshold=1e-3, check_every=10, return_n_iters=True, allow_tf32=True)
    assert 3 <= k <= 62
    assert (k - 2) % 10 == 0 or k == 62  # stops only at a check boundary (init + loop steps + extrapolation)
    assert torch.isfinite(f).all() and torch.isfinite(g).all()
    fh, gh = f - (x**2).sum(1), g - (y**2).sum(1)
    ones = torch.ones(m, d, device="cuda")
    row_mass = apply_plan_mat_flashstyle(x, y, fh, gh, log_weights(a), log_weights(b), ones, eps=eps, axis=1,
                                         allow_tf32=True)[:, 0]
    total = row_mass.sum().item()
    # with |x-y|^2 ~ 400 >> rho = 1 it is cheaper to destroy mass than to move it: the relaxed plan carries
    # (almost) no mass, and never more than the larger input mass
    assert torch.isfinite(row_mass).all() and (row_mass >= 0).all()
    assert 0.0 <= total < 1.3 + 1e-3


def test_config3_shape_annealed_alternating_block_sparse_subsample():
    """Config 3's recipe (64-component mixture in 3-D, sorted by component, annealed alternating solve, tile
    pairs kept where component centres are closer than 0.5) on a 65,536-point subsample: the block-sparse
    solve is finite and close to the dense solve where the dropped tiles carry no mass."""
    from flash_sinkhorn_b200.kernels._common import epsilon_schedule, max_diameter
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    rng = np.random.default_rng(2)
    n = m = 65536
    centres = rng.uniform(-1, 1, (64, 3))
    lx, ly = np.sort(rng.integers(0, 64, n)), np.sort(rng.integers(0, 64, m))
    x = torch.tensor(centres[lx] + 0.05 * rng.standard_normal((n, 3)), dtype=torch.float32).cuda()
    y = torch.tensor(centres[ly] + 0.05 * rng.standard_normal((m, 3)), dtype=torch.float32).cuda()
    a, b = torch.full((n,), 1.0 / n).cuda(), torch.full((m,), 1.0 / m).cuda()
    sched = epsilon_schedule(max_diameter(x, y), 0.05, 0.5)
    # tile (I, J) kept iff some component present in x-tile I is within 0.5 of some component in y-tile J
    tx, ty = (n + 127) // 128, (m + 127) // 128
    near = np.linalg.norm(centres[:, None] - centres[None], axis=-1) < 0.5
    cx = [np.unique(lx[i * 128:(i + 1) * 128]) for i in range(tx)]
    cy = [np.unique(ly[j * 128:(j + 1) * 128]) for j in range(ty)]
    px = np.zeros((tx, 64), bool)
    py = np.zeros((ty, 64), bool)
    for i, c in enumerate(cx):
        px[i, c] = True
    for j, c in enumerate(cy):
        py[j, c] = True
    mask = (px.astype(np.float32) @ near.astype(np.float32) @ py.T.astype(np.float32)) > 0
    density = mask.mean()
    assert 0.02 < density < 0.6
    fs, gs = sinkhorn_flashstyle_alternating(x, y, a, b, eps_list=sched, iters_per_eps=2, allow_tf32=False,
                                             tile_mask=torch.as_tensor(mask))
    assert torch.isfinite(fs).all() and torch.isfinite(gs).all()
    # One Gauss-Seidel iteration at the final temperature from zero potentials: dropped tiles are at least
    # (0.5 - 6 sigma)^2 = 0.04 away, i.e. exp(-0.04/eps) = e^-16 of an in-cluster weight, so the block-sparse
    # soft-min equals the dense one far below fp32 resolution of the potentials.
    eps = sched[-1]
    fd1, gd1 = sinkhorn_flashstyle_alternating(x, y, a, b, eps=eps, n_iters=1, allow_tf32=False)
    fs1, gs1 = sinkhorn_flashstyle_alternating(x, y, a, b, eps=eps, n_iters=1, allow_tf32=False,
                                               tile_mask=torch.as_tensor(mask))
    assert (fs1 - fd1).abs().max().item() < 1e-4 and (gs1 - gd1).abs().max().item() < 1e-4
