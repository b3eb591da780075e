"""N > 1 path on CPU: the row-sharded solver loop (flash_sinkhorn_b200.distributed) run as two gloo ranks,
with the dense oracle standing in for the CUDA step, must reproduce the unsharded oracle solve exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_golden
from oracle import dense_sinkhorn as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, cases, out_dir):
    """Runs the given cases with their steps interleaved (one case = the plain one-problem loop)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_sinkhorn_b200.distributed import run_many, sharded_steps, shard_layout, shard_range
        import flash_sinkhorn_b200.distributed as D
        # small alignment so that two ranks really split these ~100-row clouds
        D.SHARD_ALIGN = 8
        D.shard_layout.__defaults__ = (8,)
        D.shard_range.__defaults__ = (8,)
        built = [_build(case, rank, world, sharded_steps, shard_layout, shard_range) for case in cases]
        results = run_many([g for g, _ in built])
        for i, ((_, fin), res) in enumerate(zip(built, results)):
            np.savez(os.path.join(out_dir, f"rank{rank}_{i}.npz"), **fin(res))
    finally:
        dist.destroy_process_group()


def _build(case, rank, world, sharded_steps, shard_layout, shard_range):
    z = load_golden("solvers_small")
    x, y = z["x"].astype(np.float64), z["y"].astype(np.float64)
    a, b = z["a"].astype(np.float64), z[case["b"]].astype(np.float64)
    if case.get("self"):
        y, b = x, a
    n, m = x.shape[0], y.shape[0]
    cs, rx, ry = case["cs"], case["rho_x"], case["rho_y"]
    alpha, beta = cs * O.sqnorm(x), cs * O.sqnorm(y)
    la, lb = O.log_weights(a), O.log_weights(b)

    def step_fn(f_old, g_old, f_new, g_new, eps, w, rng):
        f_lo, f_hi, g_lo, g_hi = rng
        fo, go = f_old[:n].numpy(), g_old[:m].numpy()
        df, dg = O.dampening(eps, rx), O.dampening(eps, ry)
        cf = O.lse_update_fused(x[f_lo:f_hi], y, go, lb, eps, cs, df)   # only this rank's rows
        cg = O.lse_update_fused(y[g_lo:g_hi], x, fo, la, eps, cs, dg)
        nf = (1 - w) * fo[f_lo:f_hi] + w * cf - (w * alpha[f_lo:f_hi] * (1 - df) if df < 1 else 0.0)
        ng = (1 - w) * go[g_lo:g_hi] + w * cg - (w * beta[g_lo:g_hi] * (1 - dg) if dg < 1 else 0.0)
        f_new[f_lo:f_hi] = torch.from_numpy(nf)
        g_new[g_lo:g_hi] = torch.from_numpy(ng)

    def gather_fn(buf, shard):
        dist.all_gather_into_tensor(buf, buf[rank * shard:(rank + 1) * shard].clone())

    assert shard_layout(n, world) * world >= n and shard_range(n, world, world - 1)[1] == n
    gen = sharded_steps(
        n, m, torch.from_numpy(-alpha), torch.from_numpy(-beta), case["eps_list"],
        last_extrapolation=True, threshold=case["threshold"], check_every=case["check_every"],
        world=world, rank=rank, step_fn=step_fn, gather_fn=gather_fn, self_problem=bool(case.get("self")))

    def finish(res):
        fh, gh, fp, gp, steps = res
        return dict(f=fh.numpy() + alpha, g=gh.numpy() + beta, f_pre=fp.numpy() + alpha,
                    g_pre=gp.numpy() + beta, steps=steps)

    return gen, finish


CASES = {
    "unbalanced_schedule": dict(b="b", cs=1.0, rho_x=1.0, rho_y=4.0, threshold=None, check_every=5, eps_list=None),
    "early_stop": dict(b="b_normalised", cs=1.0, rho_x=None, rho_y=None, threshold=1e-3, check_every=4,
                       eps_list=[5.0] * 60),
    # OT(a, a): only the f half runs on each rank, g aliases f
    "self_transport": dict(b="b", cs=1.0, rho_x=None, rho_y=None, threshold=None, check_every=5, eps_list=None,
                           self=True),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_two_rank_sharded_loop_equals_unsharded_oracle(tmp_path, name):
    case = dict(CASES[name])
    z = load_golden("solvers_small")
    if case["eps_list"] is None:
        case["eps_list"] = [float(e) for e in z["sched"]]
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), [case], str(tmp_path)), nprocs=world, join=True)
    _check(tmp_path, 0, name, case, z, world)


def test_interleaved_problems_equal_one_at_a_time(tmp_path):
    """Three problems with different schedule lengths stepped round-robin (what the multi-GPU divergence
    does): each must come out exactly as when solved alone."""
    z = load_golden("solvers_small")
    names = ["unbalanced_schedule", "self_transport", "early_stop"]
    cases = []
    for nm in names:
        c = dict(CASES[nm])
        if c["eps_list"] is None:
            c["eps_list"] = [float(e) for e in z["sched"]]
        cases.append(c)
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), cases, str(tmp_path)), nprocs=world, join=True)
    for i, (nm, c) in enumerate(zip(names, cases)):
        _check(tmp_path, i, nm, c, z, world)


def _check(tmp_path, idx, name, case, z, world):
    x, y = z["x"].astype(np.float64), z["y"].astype(np.float64)
    a, b = z["a"].astype(np.float64), z[case["b"]].astype(np.float64)
    if case.get("self"):
        y, b = x, a
    want = O.solve_symmetric(x, y, a, b, case["eps_list"], cost_scale=case["cs"], rho_x=case["rho_x"],
                             rho_y=case["rho_y"], threshold=case["threshold"], check_every=case["check_every"])
    ranks = [np.load(tmp_path / f"rank{r}_{idx}.npz") for r in range(world)]
    for r in ranks:
        assert int(r["steps"]) == want["n_iters"]
        for k in ("f", "g", "f_pre", "g_pre"):
            np.testing.assert_allclose(r[k], want[k], rtol=1e-12, atol=1e-12)
    for k in ("f", "g"):
        assert np.array_equal(ranks[0][k], ranks[1][k])  # every rank ends with identical vectors
    if name == "early_stop":
        assert want["n_iters"] < 62
    # matches the fixture the reference produced for the same solve
    if name == "unbalanced_schedule":
        assert np.abs(ranks[0]["f"] - z["sym_unbal_fused_f"]).max() / np.abs(z["sym_unbal_fused_f"]).max() < 3e-5


# ---------------------------------------------------------------- alternating (Gauss-Seidel) solver
ALT_CASES = {
    "geomloss_damped": dict(b="b", cs=0.5, rho_x=1.0, rho_y=None, ott=False, threshold=None, check_every=5,
                            eps_list=[0.8], iters=12),
    "ott_balanced": dict(b="b_normalised", cs=1.0, rho_x=None, rho_y=None, ott=True, threshold=None, check_every=5,
                         eps_list=[0.6], iters=9),
    "annealed_early_stop": dict(b="b_normalised", cs=1.0, rho_x=None, rho_y=None, ott=False, threshold=1e-3,
                                check_every=3, eps_list=[8.0, 4.0, 2.0], iters=40),
    # rows split by (synthetic) kept-tile counts instead of evenly: unequal ranges, padded gather
    "uneven_ranges": dict(b="b_normalised", cs=1.0, rho_x=None, rho_y=2.0, ott=False, threshold=1e-3,
                          check_every=3, eps_list=[4.0, 1.0], iters=15, uneven=True),
    "uneven_ranges_ott": dict(b="b_normalised", cs=0.5, rho_x=None, rho_y=None, ott=True, threshold=None,
                              check_every=5, eps_list=[0.6], iters=7, uneven=True),
}


def _alt_worker(rank, world, port, case, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import flash_sinkhorn_b200.distributed as D
        D.SHARD_ALIGN = 8
        D.shard_layout.__defaults__ = (8,)
        D.shard_range.__defaults__ = (8,)
        z = load_golden("solvers_small")
        x, y = z["x"].astype(np.float64), z["y"].astype(np.float64)
        a, b = z["a"].astype(np.float64), z[case["b"]].astype(np.float64)
        n, m = x.shape[0], y.shape[0]
        cs, rx, ry, ott = case["cs"], case["rho_x"], case["rho_y"], case["ott"]
        alpha, beta = cs * O.sqnorm(x), cs * O.sqnorm(y)
        la, lb = O.log_weights(a), O.log_weights(b)
        calls = []

        def half_fn(side, f_cur, g_cur, out, eps, rng):
            lo, hi = rng
            calls.append(side)
            assert out.data_ptr() not in (f_cur.data_ptr(), g_cur.data_ptr())
            if side == "f":
                pot, logw_in, rows, cols, damp, logw_out = g_cur[:m].numpy(), lb, x[lo:hi], y, O.dampening(eps, rx), la
            else:
                pot, logw_in, rows, cols, damp, logw_out = f_cur[:n].numpy(), la, y[lo:hi], x, O.dampening(eps, ry), lb
            if ott:
                new = eps * logw_out[lo:hi] + O.lse_update_fused(rows, cols, pot, np.zeros_like(logw_in), eps, cs, damp)
            else:
                new = O.lse_update_fused(rows, cols, pot, logw_in, eps, cs, damp)
            out[lo:hi] = torch.from_numpy(new)

        def gather_fn(buf, shard):
            dist.all_gather_into_tensor(buf, buf[rank * shard:(rank + 1) * shard].clone())

        ranges = None
        if case.get("uneven"):  # explicit, unequal row ranges as a block-sparse pass gets them (8-row blocks here)
            nb, mb = -(-n // 8), -(-m // 8)
            rp_f = np.concatenate([[0], np.cumsum(1 + np.arange(nb) ** 2)])
            rp_g = np.concatenate([[0], np.cumsum(1 + (np.arange(mb)[::-1] % 7))])
            ranges = {"f": D.balanced_tile_ranges(rp_f, n, world, tile=8),
                      "g": D.balanced_tile_ranges(rp_g, m, world, tile=8)}
            assert ranges["f"][0][1] - ranges["f"][0][0] != ranges["f"][1][1] - ranges["f"][1][0]
        fh, gh, used = D.run_alternating_sharded(
            n, m, torch.from_numpy(-alpha), torch.from_numpy(-beta), case["eps_list"], case["iters"],
            ott_convention=ott, threshold=case["threshold"], check_every=case["check_every"], world=world, rank=rank,
            half_fn=half_fn, gather_fn=gather_fn, ranges=ranges)
        assert calls[:2] == (["g", "f"] if ott else ["f", "g"]) and len(calls) == 2 * used
        np.savez(os.path.join(out_dir, f"alt_rank{rank}.npz"), f=fh.numpy() + alpha, g=gh.numpy() + beta, used=used)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", sorted(ALT_CASES))
def test_two_rank_alternating_loop_equals_unsharded_oracle(tmp_path, name):
    case = ALT_CASES[name]
    world = 2
    mp.spawn(_alt_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)
    z = load_golden("solvers_small")
    x, y = z["x"].astype(np.float64), z["y"].astype(np.float64)
    a, b = z["a"].astype(np.float64), z[case["b"]].astype(np.float64)
    want = O.solve_alternating(x, y, a, b, case["eps_list"], case["iters"], cost_scale=case["cs"],
                               rho_x=case["rho_x"], rho_y=case["rho_y"], ott_convention=case["ott"],
                               threshold=case["threshold"], check_every=case["check_every"])
    ranks = [np.load(tmp_path / f"alt_rank{r}.npz") for r in range(world)]
    for r in ranks:
        assert int(r["used"]) == want["n_iters"]
        np.testing.assert_allclose(r["f"], want["f"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(r["g"], want["g"], rtol=1e-12, atol=1e-12)
    assert np.array_equal(ranks[0]["f"], ranks[1]["f"]) and np.array_equal(ranks[0]["g"], ranks[1]["g"])
    if name == "annealed_early_stop":
        assert want["n_iters"] < 120


def test_balanced_tile_ranges_cover_the_rows_and_balance_the_kept_tiles():
    import flash_sinkhorn_b200.distributed as D
    rng = np.random.default_rng(0)
    for nblk, world in [(1, 2), (7, 4), (64, 8), (7813, 8), (100, 3)]:
        counts = rng.integers(0, 50, size=nblk)
        counts[rng.integers(0, nblk)] += 1  # at least one kept tile
        rp = np.concatenate([[0], np.cumsum(counts)])
        rows = nblk * 128 - 37
        ranges = D.balanced_tile_ranges(rp, rows, world)
        assert len(ranges) == world and ranges[0][0] == 0 and ranges[-1][1] == rows
        for (lo, hi), (lo2, _) in zip(ranges, ranges[1:]):
            assert hi == lo2 and lo % 128 == 0 and lo <= hi
        per_rank = [int(rp[-(-hi // 128)] - rp[lo // 128]) for lo, hi in ranges]
        assert sum(per_rank) == rp[-1]
        # no rank exceeds the ideal share by more than one block's worth of tiles
        assert max(per_rank) <= rp[-1] / world + counts.max()


# ---------------------------------------------------------------- fused lockstep schedule (packed potentials)
def _fused_worker(rank, world, port, cases, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import flash_sinkhorn_b200.distributed as D
        D.SHARD_ALIGN = 8
        D.shard_layout.__defaults__ = (8,)
        D.shard_range.__defaults__ = (8,)
        z = load_golden("solvers_small")
        data, problems = [], []
        for case in cases:
            x, y = z["x"].astype(np.float64), z["y"].astype(np.float64)
            a, b = z["a"].astype(np.float64), z[case["b"]].astype(np.float64)
            if case.get("self"):
                y, b = x, a
            cs = case["cs"]
            alpha, beta = cs * O.sqnorm(x), cs * O.sqnorm(y)
            data.append(dict(x=x, y=y, la=O.log_weights(a), lb=O.log_weights(b), alpha=alpha, beta=beta, cs=cs,
                             rx=case["rho_x"], ry=case["rho_y"]))
            problems.append(dict(n=x.shape[0], m=y.shape[0], f_hat0=torch.from_numpy(-alpha),
                                 g_hat0=torch.from_numpy(-beta), eps_list=case["eps_list"], last_extrapolation=True,
                                 threshold=case["threshold"], check_every=case["check_every"],
                                 self_problem=bool(case.get("self"))))
        calls = []

        def step_fn(items, old, new, layout):
            calls.append(len(items))
            mine = new.view(world, layout.width)[rank]
            for k, eps, w, (f_lo, f_hi, g_lo, g_hi) in items:
                dk = data[k]
                fo, go = layout.full(old, k, 0).numpy(), layout.full(old, k, 1).numpy()
                df, dg = O.dampening(eps, dk["rx"]), O.dampening(eps, dk["ry"])
                (f_off, f_shard, _), (g_off, g_shard, _) = layout.slots[k]
                if f_hi > f_lo:
                    cf = O.lse_update_fused(dk["x"][f_lo:f_hi], dk["y"], go, dk["lb"], eps, dk["cs"], df)
                    nf = (1 - w) * fo[f_lo:f_hi] + w * cf - (w * dk["alpha"][f_lo:f_hi] * (1 - df) if df < 1 else 0.0)
                    mine[f_off:f_off + (f_hi - f_lo)] = torch.from_numpy(nf)
                if g_hi > g_lo:
                    cg = O.lse_update_fused(dk["y"][g_lo:g_hi], dk["x"], fo, dk["la"], eps, dk["cs"], dg)
                    ng = (1 - w) * go[g_lo:g_hi] + w * cg - (w * dk["beta"][g_lo:g_hi] * (1 - dg) if dg < 1 else 0.0)
                    mine[g_off:g_off + (g_hi - g_lo)] = torch.from_numpy(ng)

        def gather_fn(buf, width):
            dist.all_gather_into_tensor(buf, buf[rank * width:(rank + 1) * width].clone())

        results = D.run_symmetric_fused(problems, world=world, rank=rank, step_fn=step_fn, gather_fn=gather_fn)
        assert max(calls) == len(cases) and min(calls) >= 1  # every step of all live problems in one call
        for i, ((fh, gh, fp, gp, steps), dk) in enumerate(zip(results, data)):
            np.savez(os.path.join(out_dir, f"rank{rank}_{i}.npz"), f=fh.numpy() + dk["alpha"], g=gh.numpy() + dk["beta"],
                     f_pre=fp.numpy() + dk["alpha"], g_pre=gp.numpy() + dk["beta"], steps=steps)
    finally:
        dist.destroy_process_group()


def test_fused_lockstep_schedule_equals_one_at_a_time(tmp_path):
    """The multi-GPU debiased divergence steps its three problems in lockstep, one fused launch and one all-gather
    of a packed buffer per step: problems of different schedule lengths, a self-transport one and an early stop
    must each come out exactly as when solved alone."""
    z = load_golden("solvers_small")
    names = ["unbalanced_schedule", "self_transport", "early_stop"]
    cases = []
    for nm in names:
        c = dict(CASES[nm])
        if c["eps_list"] is None:
            c["eps_list"] = [float(e) for e in z["sched"]]
        cases.append(c)
    world = 2
    mp.spawn(_fused_worker, args=(world, _free_port(), cases, str(tmp_path)), nprocs=world, join=True)
    for i, (nm, c) in enumerate(zip(names, cases)):
        _check(tmp_path, i, nm, c, z, world)
