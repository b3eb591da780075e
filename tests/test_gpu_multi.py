"""Two-GPU check of the row-sharded solver and gradient (NCCL): results equal the single-GPU ones.
Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flash_sinkhorn_b200 import SamplesLoss
        gen = torch.Generator().manual_seed(3)
        n, m, d = 3000, 2500, 64
        x = torch.randn(n, d, generator=gen).cuda().requires_grad_(True)
        y = (0.3 + torch.randn(m, d, generator=gen)).cuda()
        for tf32 in (True, False):
            loss = SamplesLoss("sinkhorn", blur=0.3, scaling=0.7, debias=True, allow_tf32=tf32,
                               threshold=1e-4, inner_iterations=3, process_group=dist.group.WORLD)
            val = loss(x, y)
            (gx,) = torch.autograd.grad(val, x)
            torch.cuda.synchronize()
            np.savez(os.path.join(out_dir, f"r{rank}_{int(tf32)}.npz"), loss=val.item(), gx=gx.cpu().numpy())
        # large feature dimension (K-streamed kernels, gradient through the weight matrix), semi-unbalanced
        xl, yl = _large_d_clouds()
        xl = xl.cuda().requires_grad_(True)
        loss = SamplesLoss("sinkhorn", blur=0.3, reach_x=1.0, half_cost=True, use_epsilon_scaling=False, eps=0.09,
                           n_iters=8, process_group=dist.group.WORLD)
        val = loss(xl, yl.cuda())
        (gx,) = torch.autograd.grad(val, xl)
        np.savez(os.path.join(out_dir, f"r{rank}_large_d.npz"), loss=val.item(), gx=gx.cpu().numpy())
        # block-sparse annealed alternating solve, rows split over the ranks by kept tiles
        from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
        xs, ys, a, b, mask = _sparse_problem()
        f, g = sinkhorn_flashstyle_alternating(xs.cuda(), ys.cuda(), a.cuda(), b.cuda(), eps_list=[0.5, 0.1],
                                               iters_per_eps=3, tile_mask=mask, process_group=dist.group.WORLD)
        np.savez(os.path.join(out_dir, f"r{rank}_tiles.npz"), f=f.cpu().numpy(), g=g.cpu().numpy())
    finally:
        dist.destroy_process_group()


def _large_d_clouds():
    gen = torch.Generator().manual_seed(8)
    return (torch.nn.functional.normalize(torch.randn(900, 700, generator=gen), dim=1),
            torch.nn.functional.normalize(torch.randn(1100, 700, generator=gen), dim=1))


def _sparse_problem():
    gen = torch.Generator().manual_seed(9)
    n, m = 2000, 1700
    x, y = torch.rand(n, 3, generator=gen), torch.rand(m, 3, generator=gen)
    mask = torch.rand((n + 127) // 128, (m + 127) // 128, generator=gen) < 0.4
    mask[:, 0] = True
    mask[0, :] = True
    mask[3:6, 1:] = False  # few tiles in these row blocks: the kept-tile split is far from the row split
    return x, y, torch.full((n,), 1.0 / n), torch.full((m,), 1.0 / m), mask


def test_sharded_two_gpu_equals_single_gpu(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from flash_sinkhorn_b200 import SamplesLoss
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    gen = torch.Generator().manual_seed(3)
    n, m, d = 3000, 2500, 64
    x = torch.randn(n, d, generator=gen).cuda().requires_grad_(True)
    y = (0.3 + torch.randn(m, d, generator=gen)).cuda()
    for tf32 in (True, False):
        loss = SamplesLoss("sinkhorn", blur=0.3, scaling=0.7, debias=True, allow_tf32=tf32, threshold=1e-4,
                           inner_iterations=3)
        val = loss(x, y)
        (gx,) = torch.autograd.grad(val, x)
        want = gx.cpu().numpy()
        for r in range(world):
            z = np.load(tmp_path / f"r{r}_{int(tf32)}.npz")
            assert abs(float(z["loss"]) - val.item()) <= 1e-5 * abs(val.item())
            # same kernels, but the column split (hence the merge order of partial sums) depends on the
            # number of row blocks per rank: agreement is to rounding, amplified by the solve
            assert np.abs(z["gx"] - want).max() <= (2e-3 if tf32 else 2e-4) * np.abs(want).max()
        z0, z1 = (np.load(tmp_path / f"r{r}_{int(tf32)}.npz") for r in range(2))
        assert np.array_equal(z0["gx"], z1["gx"])  # all ranks hold identical results
    # large d: K-streamed passes and the weight-matrix gradient, sharded vs single GPU
    xl, yl = _large_d_clouds()
    xl = xl.cuda().requires_grad_(True)
    loss = SamplesLoss("sinkhorn", blur=0.3, reach_x=1.0, half_cost=True, use_epsilon_scaling=False, eps=0.09, n_iters=8)
    val = loss(xl, yl.cuda())
    (gx,) = torch.autograd.grad(val, xl)
    for r in range(world):
        z = np.load(tmp_path / f"r{r}_large_d.npz")
        assert abs(float(z["loss"]) - val.item()) <= 1e-5 * abs(val.item())
        assert np.abs(z["gx"] - gx.cpu().numpy()).max() <= 2e-3 * np.abs(gx.cpu().numpy()).max()
    # block-sparse alternating solve: split by kept tiles vs single GPU
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    xs, ys, a, b, mask = _sparse_problem()
    f, g = sinkhorn_flashstyle_alternating(xs.cuda(), ys.cuda(), a.cuda(), b.cuda(), eps_list=[0.5, 0.1], iters_per_eps=3,
                                           tile_mask=mask)
    for r in range(world):
        z = np.load(tmp_path / f"r{r}_tiles.npz")
        assert np.abs(z["f"] - f.cpu().numpy()).max() <= 2e-3 * np.abs(f.cpu().numpy()).max()
        assert np.abs(z["g"] - g.cpu().numpy()).max() <= 2e-3 * np.abs(g.cpu().numpy()).max()
    z0, z1 = (np.load(tmp_path / f"r{r}_tiles.npz") for r in range(2))
    assert np.array_equal(z0["f"], z1["f"]) and np.array_equal(z0["g"], z1["g"])
