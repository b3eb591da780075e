#!/usr/bin/env python
"""Headline benchmark: headline configuration 2 (n = m = 50,000, d = 64, eps = 0.01, 100 fixed symmetric
iterations, debiased, forward + analytic grad_x) on N B200 GPUs of one node.

    python bench.py [--gpus N --steps K --warmup W] [--impl reference] [--n 50000 --d 64]

A "step" is one full SamplesLoss forward + backward on one synthetic problem. Prints ONE JSON line
(rank 0). `value` = cost-matrix entries evaluated per second over all ranks with inputs resident in
HBM; `e2e` = same metric through the public API with pinned HOST buffers, copies included.
Multi-GPU (torchrun, one rank per GPU): the SAME problem is solved by all ranks together - rows of every
potential update and of the gradient are sharded over the ranks and all-gathered over NCCL after each
half-step ("strong" scaling: total work fixed, `value` counts every entry once).
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def entries_per_step(n, m, n_iters, debias=True):
    """Score-matrix entries evaluated by one forward+grad_x step (one exp and one d-long dot each).
    Cross term: (n_iters + 2) Jacobi steps x 2 soft-mins; gradient: one pass per requested side.
    Self terms OT(x,x), OT(y,y): both potentials are equal at every step, so the engine evaluates ONE
    soft-min per step (the reference evaluates two; results are bit-identical)."""
    steps = n_iters + 2
    e = 2 * steps * n * m + n * m                      # OT(x,y) + grad_x
    if debias:
        e += steps * n * n + 2 * n * n                 # OT(x,x): x enters twice -> both gradient sides
        e += steps * m * m                             # OT(y,y): no gradient w.r.t. x
    return e


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_sample(n, m, d, eps, seconds_budget=20.0):
    """Dense PyTorch CPU baseline on a bounded sample of the same workload (entries/s is scale-free)."""
    import torch
    from oracle import dense_torch
    # all host threads, also under torchrun (which exports OMP_NUM_THREADS=1 to every rank when N > 1)
    torch.set_num_threads(max(torch.get_num_threads(), len(os.sched_getaffinity(0))))
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(n, d, generator=gen)
    y = 0.5 + torch.randn(m, d, generator=gen)
    a, b = torch.full((n,), 1.0 / n), torch.full((m,), 1.0 / m)
    # one Jacobi step at full size costs 2*n*m entries at ~2e8 entries/s on 8 cores: bound the row count
    rows = n
    target_entries = 2.0e8 * seconds_budget / 2  # init step + 1 loop step
    if 2.0 * rows * m > target_entries:
        rows = max(1024, int(target_entries / (2.0 * m)))
    xs, a_s = x[:rows], torch.full((rows,), 1.0 / rows)
    _, _, dt, ent = dense_torch.symmetric_steps(xs, y, a_s, b, eps, 1)
    return {"value": ent / dt, "unit": "entries/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"init + 1 Jacobi step of the dense fp32 log-domain solve on {rows} x {m} x {d} "
                      f"(row-chunked, {dt:.1f} s)"}, dt, ent


# ---------------------------------------------------------------------------------------------------------
# The other benchmark configurations (--config 3 | 3csr | 4 | 5). Same contract line; the default run is config 2.
# ---------------------------------------------------------------------------------------------------------
def make_config3(n, seed=2):
    """64-component Gaussian mixture in 3-D (centres U[-1,1]^3, std 0.05), points sorted by component."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    centres = torch.rand(64, 3, generator=gen) * 2 - 1
    out = []
    for _ in range(2):
        lab = torch.sort(torch.randint(0, 64, (n,), generator=gen)).values
        out.append((centres[lab] + 0.05 * torch.randn(n, 3, generator=gen), lab))
    return centres, out[0], out[1]


def config3_tile_mask(centres, lab_x, lab_y, n, m, radius=0.5):
    """Keep a 128 x 128 tile pair when some component present in the row tile and some component present in the
    column tile have centres closer than `radius` (labels are sorted, so a tile holds a contiguous label range)."""
    import torch
    near = (torch.cdist(centres, centres) < radius).to(torch.int32)
    pre = torch.zeros(65, 65, dtype=torch.int32)
    pre[1:, 1:] = near.cumsum(0).cumsum(1)

    def ranges(lab, rows):
        nt = (rows + 127) // 128
        lo = lab[::128][:nt]
        hi = lab[torch.clamp(torch.arange(nt) * 128 + 127, max=rows - 1)]
        return lo.long(), hi.long() + 1

    xl, xh = ranges(lab_x, n)
    yl, yh = ranges(lab_y, m)
    cnt = pre[xh][:, yh] - pre[xl][:, yh] - pre[xh][:, yl] + pre[xl][:, yl]
    return cnt > 0


def pass_ms_by_difference(run_solve, k1, k2, reps=3):
    """Device time of ONE soft-min pass inside a symmetric solve: (T(k2 iterations) - T(k1 iterations)) divided by
    the 2 (k2 - k1) passes the longer solve adds. Staging, norms and Python overhead are common to both and drop
    out; the per-pass bias kernel stays in (it is part of every pass)."""
    import torch
    times = []
    for k in (k1, k2):
        run_solve(k)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run_solve(k)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / reps)
    return (times[1] - times[0]) / (2.0 * (k2 - k1))


def bench_extra(args):
    """Configs 3 (annealed alternating, 1e6 x 1e6 x 3, dense or block-sparse), 4 (unbalanced, early stop, gradient,
    20-iteration HVP at 100k x 80k x 128) and 5 (semi-unbalanced, 16384^2 x 2048, forward + grad_x)."""
    import torch
    import torch.distributed as dist
    from flash_sinkhorn_b200 import SamplesLoss, _lib
    from flash_sinkhorn_b200.kernels._common import epsilon_schedule, max_diameter
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse_fused
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating, sinkhorn_flashstyle_symmetric

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD if world > 1 else None
    lib = _lib.load()
    cfg = args.config
    tf32 = not args.fp32
    extra = {}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()


    # ---- per-config workload: pinned host inputs, a resident step, an end-to-end step, the entry count ----
    if cfg in ("3", "3csr"):
        n = m = args.n if args.n is not None else 1000000
        d = 3
        centres, (xh, lx), (yh, ly) = make_config3(n)
        host_in = [xh.pin_memory(), yh.pin_memory()]
        a_w = torch.full((n,), 1.0 / n, device=dev)
        b_w = torch.full((m,), 1.0 / m, device=dev)
        sched = epsilon_schedule(max_diameter(xh, yh), 0.01, 0.5)
        mask = config3_tile_mask(centres, lx, ly, n, m) if cfg == "3csr" else None
        if mask is None:
            pass_entries = float(n) * m
        else:
            rows = torch.full((mask.shape[0],), 128.0, dtype=torch.float64)
            cols = torch.full((mask.shape[1],), 128.0, dtype=torch.float64)
            rows[-1] = n - 128 * (mask.shape[0] - 1)
            cols[-1] = m - 128 * (mask.shape[1] - 1)
            pass_entries = float(rows @ mask.double() @ cols)
            extra["tile_density"] = float(mask.double().mean())
        iters_per = 10
        per_step = 2.0 * iters_per * len(sched) * pass_entries
        workload = (f"config3{'csr' if mask is not None else ''}: annealed alternating Sinkhorn n=m={n} d=3, 64-component "
                    f"mixture sorted by component, eps from diameter^2 to 1e-4 (scaling 0.5, {len(sched)} stages x {iters_per} "
                    f"iterations){', 128x128 tiles kept where centres are closer than 0.5' if mask is not None else ''}")

        def solve(x, y, stages):
            return sinkhorn_flashstyle_alternating(x, y, a_w, b_w, eps_list=stages, iters_per_eps=iters_per,
                                                   tile_mask=mask, allow_tf32=tf32, process_group=group)

        step_resident = lambda x, y: solve(x, y, sched)
        warm_step = lambda x, y: solve(x, y, sched[:1])  # one stage (20 passes) per warm-up step
        out_host = [torch.empty(n).pin_memory(), torch.empty(m).pin_memory()]
        kernel_fn = lambda x, y: sinkhorn_flashstyle_alternating(x, y, a_w, b_w, eps=sched[-1], n_iters=2, tile_mask=mask,
                                                                 allow_tf32=tf32)
        kernel_entries, kernel_name = 4 * pass_entries, "alternating half-step (one soft-min pass), mean of 4"
        flop_per_entry = 2 * d
        kernel_timer = None
    elif cfg == "5":
        n = m = args.n if args.n is not None else 16384
        d = args.d if args.d is not None else 2048
        gen = torch.Generator().manual_seed(4)
        xh = torch.nn.functional.normalize(torch.randn(n, d, generator=gen), dim=1)
        yh = torch.nn.functional.normalize(torch.randn(m, d, generator=gen), dim=1)
        host_in = [xh.pin_memory(), yh.pin_memory()]
        iters = 50
        loss_fn = SamplesLoss("sinkhorn", blur=0.05, reach_x=1.0, reach_y=None, half_cost=True, use_epsilon_scaling=False,
                              eps=0.0025, n_iters=iters, allow_tf32=tf32, process_group=group)
        per_step = 2.0 * (iters + 2) * n * m + float(n) * m
        workload = (f"config5: semi-unbalanced Sinkhorn n=m={n} d={d}, unit-sphere rows, blur=0.05 reach_x=1 half_cost, "
                    f"{iters} fixed iterations, forward + grad_x")

        def step_resident(x, y):
            xs = x.detach().requires_grad_(True)
            val = loss_fn(xs, y)
            (gx,) = torch.autograd.grad(val, xs)
            return val, gx

        warm_step = step_resident
        out_host = [torch.empty(n, d).pin_memory()]
        lb = torch.full((m,), -math.log(m), device=dev)
        kernel_fn = lambda x, y: flashsinkhorn_lse_fused(x, y, -0.5 * (y * y).sum(1), lb, 0.0025, cost_scale=0.5,
                                                         allow_tf32=tf32)
        kernel_entries, kernel_name = float(n) * m, "row soft-min pass (K-streamed tcgen05), n*m entries per launch"
        flop_per_entry = 2 * d
        a5 = torch.full((n,), 1.0 / n, device=dev)
        kernel_timer = lambda x, y: pass_ms_by_difference(
            lambda k: sinkhorn_flashstyle_symmetric(x, y, a5, a5, use_epsilon_scaling=False, eps=0.0025, n_iters=k,
                                                    cost_scale=0.5, reach_x=1.0, last_extrapolation=False,
                                                    allow_tf32=tf32), 2, 12)
    else:  # config 4
        if world > 1:
            raise SystemExit("config 4 includes the Hessian-vector product, which is single-GPU: run it with --gpus 1")
        n, m, d = 100000, 80000, 128
        if args.n is not None:
            n, m = args.n, int(args.n * 0.8)
        gen = torch.Generator().manual_seed(3)
        xh = torch.randn(n, d, generator=gen)
        yh = 1.5 * torch.randn(m, d, generator=gen)
        a_w = torch.softmax(torch.randn(n, generator=gen), 0).to(dev)
        b_w = (1.3 * torch.softmax(torch.randn(m, generator=gen), 0)).to(dev)
        vh = torch.randn(n, d, generator=gen)
        host_in = [xh.pin_memory(), yh.pin_memory(), vh.pin_memory()]
        cg_iters = 20
        kw = dict(blur=0.2, reach=1.0, use_epsilon_scaling=False, eps=0.04, n_iters=500, threshold=1e-3)
        loss_fn = SamplesLoss("sinkhorn", normalize=False, inner_iterations=10, hvp_max_cg_iter=cg_iters,
                              allow_tf32=tf32, **kw)

        def step_resident(x, y, v):
            xs = x.detach().requires_grad_(True)
            val = loss_fn(a_w, xs, b_w, y)
            (gx,) = torch.autograd.grad(val, xs, create_graph=True)
            (hv,) = torch.autograd.grad((gx * v).sum(), xs)
            return val, gx.detach(), hv

        warm_step = step_resident
        out_host = [torch.empty(n, d).pin_memory(), torch.empty(n, d).pin_memory()]
        # steps the early stop leaves (same solve, run once outside the timed region)
        x0, y0 = xh.to(dev), yh.to(dev)
        used = sinkhorn_flashstyle_symmetric(x0, y0, a_w, b_w, check_every=10, return_n_iters=True, allow_tf32=tf32,
                                             **kw)[-1]
        del x0, y0
        extra["solver_steps_used"] = int(used)
        hvp_passes = 6 + 2 * cg_iters + 4  # the reference's launch count: vector passes, 3 matrix passes, Mat5
        per_step = (2.0 * used + 1 + hvp_passes) * n * m
        extra["entries_note"] = (f"{used} Jacobi steps x 2 soft-mins + 1 gradient pass + {hvp_passes} plan passes of the "
                                 f"HVP (reference accounting, {cg_iters} CG iterations), n*m entries each")
        workload = (f"config4: unbalanced Sinkhorn n={n} m={m} d={d}, masses 1.0/1.3, blur=0.2 reach=1, n_iters=500 "
                    f"threshold=1e-3 inner_iterations=10, loss + grad_x + HVP ({cg_iters} CG iterations)")
        la = b_w.log()
        kernel_fn = lambda x, y, v=None: flashsinkhorn_lse_fused(x, y, -(y * y).sum(1), la, 0.04, allow_tf32=tf32)
        kernel_entries, kernel_name = float(n) * m, "row soft-min pass of the solve, n*m entries per launch"
        flop_per_entry = 2 * d
        kernel_timer = lambda x, y, v=None: pass_ms_by_difference(
            lambda k: sinkhorn_flashstyle_symmetric(x, y, a_w, b_w, use_epsilon_scaling=False, eps=0.04, n_iters=k,
                                                    reach=1.0, last_extrapolation=False, allow_tf32=tf32), 2, 12)

    dev_in = [t.to(dev) for t in host_in]
    if args.kernel_only and cfg == "4":  # small runs for profilers: one step (solve, gradient, HVP), no timing loops
        outs = step_resident(*dev_in)
        torch.cuda.synchronize()
        print(json.dumps({"kernel_only": True, "config": cfg, "n": n, "m": m, "d": d, "loss": float(outs[0].detach()),
                          "hvp_norm": float(outs[2].norm())}))
        return 0
    if args.kernel_only:  # small runs for profilers: only the dominant kernel, a few launches
        for _ in range(3):
            kernel_fn(*dev_in)
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(3):
            kernel_fn(*dev_in)
        k1.record()
        torch.cuda.synchronize()
        print(json.dumps({"kernel_only": True, "config": cfg, "n": n, "m": m, "d": d, "kernel": kernel_name,
                          "kernel_ms": k0.elapsed_time(k1) / 3, "mode": "tf32" if tf32 else "fp32(3xTF32)"}))
        return 0

    def step_e2e():
        ins = [t.to(dev, non_blocking=True) for t in host_in]
        outs = step_resident(*ins)
        outs = outs if isinstance(outs, (tuple, list)) else (outs,)
        big = [o for o in outs if o.ndim > 0]
        for dst, src in zip(out_host, big):
            dst.copy_(src, non_blocking=True)
        scal = [o for o in outs if o.ndim == 0]
        return float(scal[0].item()) if scal else float(big[0][0].item())  # device->host read closes the step

    for _ in range(args.warmup):
        warm_step(*dev_in)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = lib.fs_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        outs = step_resident(*dev_in)
    e1.record()
    barrier()
    launches = lib.fs_launch_count() - launches0
    ms = e0.elapsed_time(e1)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        result = step_e2e()
    t1.record()
    barrier()
    ms_e2e = t0.elapsed_time(t1)
    clocks = sampler.stop()

    # parts of a config-4 step, timed one by one (solve with early stop / gradient / HVP)
    if cfg == "4":
        x, y, v = dev_in
        k0, k1, k2, k3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        xs = x.detach().requires_grad_(True)
        k0.record()
        val = loss_fn(a_w, xs, b_w, y)
        k1.record()
        (gx,) = torch.autograd.grad(val, xs, create_graph=True)
        k2.record()
        (hv,) = torch.autograd.grad((gx * v).sum(), xs)
        k3.record()
        torch.cuda.synchronize()
        extra.update(solve_ms=k0.elapsed_time(k1), grad_ms=k1.elapsed_time(k2), hvp_ms=k2.elapsed_time(k3))
        del gx, hv, val, xs

    # dominant kernel, timed alone on the launching stream (rank 0's GPU; single-GPU launch)
    for _ in range(3):
        kernel_fn(*dev_in)
    reps = 5
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    k0.record()
    for _ in range(reps):
        kernel_fn(*dev_in)
    k1.record()
    torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / reps
    kernel_how = "stand-alone call (includes staging of the operands), mean of 5"
    if kernel_timer is not None:  # one pass inside a solve, by differencing two solve lengths
        kernel_ms = kernel_timer(*dev_in)
        kernel_how = "inside a solve: (T(12 iterations) - T(2 iterations)) / 20 passes, CUDA events"
    barrier()

    times = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = times.tolist()
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        exp_peak = float(lib.fs_micro_exp_rate(0, 32))
        bf16 = peaks.get("bf16_tflops_sustained", 1400.0) * 1e12
        tc_flops = bf16 / 2  # TF32 dense = half the measured bf16 rate
        mult = 1 if tf32 else 3
        tc_peak_entries = tc_flops / (flop_per_entry * mult)
        achieved = kernel_entries / (kernel_ms * 1e-3)
        tensor_bound = tc_peak_entries < exp_peak
        if tensor_bound:
            roof = {"bound": "tensor", "achieved": achieved * flop_per_entry * mult / 1e12, "peak": tc_flops / 1e12,
                    "unit": "TFLOP/s", "frac": achieved * flop_per_entry * mult / tc_flops}
        else:
            roof = {"bound": "exp", "achieved": achieved, "peak": exp_peak, "unit": "entries/s", "frac": achieved / exp_peak}
        roof.update({"traffic": None, "kernel": kernel_name, "kernel_ms": kernel_ms, "kernel_timing": kernel_how,
                     "flop_per_entry": flop_per_entry * mult, "entries_per_s": achieved,
                     "peak_source": "of measured: tensor = bf16 sustained (MEASURED_PEAKS.json) / 2 for TF32; exp = "
                                    "ex2.approx rate from fs_micro_exp_rate(0,32) on this GPU"})
        total = per_step * args.steps
        h2d = sum(t.numel() * 4 for t in host_in)
        d2h = sum(t.numel() * 4 for t in out_host) + 4
        line = {
            "metric": "cost_entries_per_sec", "value": total / (ms * 1e-3), "unit": "entries/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "tf32 products, f32 accumulate/exp" if tf32 else "f32 (3xTF32 products)", "data": "synthetic",
            "config": {"workload": workload, "entries_per_step": per_step,
                       "parallelism": (f"rows sharded over {world} GPUs, all-gather per half-step" if world > 1 else "single GPU"),
                       "l2": "not flushed: operands are re-streamed from L2/HBM by design, the passes are compute-bound",
                       "result": result, **extra},
            "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "entries/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
        }
        if not args.skip_cpu and world == 1:
            cb, _, _ = cpu_reference_sample(min(n, 50000), min(m, 50000), d, 0.05, seconds_budget=10.0)
            line["cpu_baseline"] = cb
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0

def bench_reference_triton(args):
    """The UNMODIFIED reference package (its Triton kernels, JIT-compiled for this GPU) on the same workload, when an
    install of it is present under baseline/_ref. Context for the numbers of this library: the kernel to beat. Not
    part of the product; `--impl reference` (the reference's CPU path) is the arm the contract asks for."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    try:
        sys.path.insert(0, ref_dir)
        import torch
        from flash_sinkhorn import SamplesLoss as RefLoss  # noqa: the reference's own public API
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference_triton", "unavailable": f"{type(exc).__name__}: {exc}"[:200]}))
        return 0
    dev = torch.device("cuda", 0)
    cfg = args.config
    if cfg == "5":
        n = m = args.n or 16384
        d, iters, eps = args.d or 2048, 50, 0.0025
        gen = torch.Generator().manual_seed(4)
        x = torch.nn.functional.normalize(torch.randn(n, d, generator=gen), dim=1).to(dev)
        y = torch.nn.functional.normalize(torch.randn(m, d, generator=gen), dim=1).to(dev)
        loss_fn = RefLoss("sinkhorn", blur=0.05, reach_x=1.0, reach_y=None, half_cost=True, use_epsilon_scaling=False,
                          eps=eps, n_iters=iters, allow_tf32=not args.fp32)
        per_step = 2.0 * (iters + 2) * n * m + float(n) * m
        entries_ref = per_step
    else:
        n = m = args.n or 50000
        d, iters, eps = args.d or 64, args.iters, 0.01
        gen = torch.Generator().manual_seed(1)
        x = torch.randn(n, d, generator=gen).to(dev)
        y = (0.5 + torch.randn(m, d, generator=gen)).to(dev)
        loss_fn = RefLoss("sinkhorn", blur=0.1, use_epsilon_scaling=False, eps=eps, n_iters=iters, half_cost=False,
                          debias=True, allow_tf32=not args.fp32)
        per_step = entries_per_step(n, m, iters, True)
        # the reference evaluates both soft-mins of the self terms: what it actually computes per step
        entries_ref = 2 * (iters + 2) * (n * m + n * n + m * m) + n * m + 2 * n * n

    def step():
        xs = x.detach().requires_grad_(True)
        val = loss_fn(xs, y)
        (gx,) = torch.autograd.grad(val, xs)
        return val

    for _ in range(max(1, args.warmup)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        val = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"impl": "reference_triton", "metric": "cost_entries_per_sec", "value": per_step / (ms * 1e-3),
                      "unit": "entries/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                      "config": {"workload": f"config{cfg}: n=m={n} d={d} eps={eps} n_iters={iters}, stock SamplesLoss "
                                             "of the reference package (Triton JIT on this GPU), forward + grad_x",
                                 "entries_counted": per_step, "entries_the_reference_evaluates": entries_ref,
                                 "loss": float(val)},
                      "dtype": "fp32 (allow_tf32=False)" if args.fp32 else "tf32 (reference default)"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_triton"])
    ap.add_argument("--config", default="2", choices=["2", "3", "3csr", "4", "5"],
                    help="benchmark configuration (default 2, the one the headline metric is quoted on)")
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--d", type=int, default=None)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--no-debias", action="store_true")
    ap.add_argument("--fp32", action="store_true", help="3xTF32 exact-fp32 mode instead of TF32")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only time the dominant kernels (one LSE pass, one gradient pass); small, for profilers")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = {"2": 3, "3": 1, "3csr": 1, "4": 1, "5": 3}[args.config]
    if args.impl == "reference_triton":
        return bench_reference_triton(args)
    if args.config != "2" and args.impl == "b200":
        return bench_extra(args)
    if args.n is None:
        args.n = 50000
    if args.d is None:
        args.d = 64

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n = m = args.n
    d, eps, iters = args.d, 0.01, args.iters
    debias = not args.no_debias
    workload = (f"config2: symmetric Sinkhorn n=m={n} d={d} eps={eps} n_iters={iters} fixed-eps "
                f"{'debiased ' if debias else ''}forward+grad_x, x~N(0,1) y~N(0.5,1), uniform weights")
    per_step = entries_per_step(n, m, iters, debias)

    if args.impl == "reference":
        if rank != 0:
            return 0
        vals = []
        for i in range(args.warmup + args.steps):
            cb, dt, ent = cpu_reference_sample(n, m, d, eps, seconds_budget=12.0)
            if i >= args.warmup:
                vals.append((ent, dt))
        ent = sum(v[0] for v in vals)
        dt = sum(v[1] for v in vals)
        cb["value"] = ent / dt
        line = {"impl": "reference", "metric": "cost_entries_per_sec", "value": ent / dt, "unit": "entries/s",
                "n_gpus": 0, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": {"workload": workload, "note": "each step = bounded sample: " + cb["sample"]},
                "cpu_baseline": cb,
                "e2e": {"value": ent / dt, "unit": "entries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist
    from flash_sinkhorn_b200 import SamplesLoss, _lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    group = dist.group.WORLD if world > 1 else None
    gen = torch.Generator().manual_seed(1)  # identical inputs on every rank (replicated clouds)
    x_host = torch.randn(n, d, generator=gen).pin_memory()
    y_host = (0.5 + torch.randn(m, d, generator=gen)).pin_memory()
    gx_host = torch.empty(n, d).pin_memory()
    loss_fn = SamplesLoss("sinkhorn", blur=0.1, use_epsilon_scaling=False, eps=eps, n_iters=iters,
                          half_cost=False, debias=debias, allow_tf32=not args.fp32, process_group=group)

    if args.kernel_only:
        from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid
        from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse_fused
        from flash_sinkhorn_b200 import c_transform_fwd
        x_dev, y_dev = x_host.to(dev), y_host.to(dev)
        gh = -(y_dev**2).sum(1)
        a_w = torch.full((n,), 1.0 / n, device=dev)
        b_w = torch.full((m,), 1.0 / m, device=dev)
        lb = b_w.log()
        res = {}
        for name, fn in (("lse_pass", lambda: flashsinkhorn_lse_fused(x_dev, y_dev, gh, lb, eps, allow_tf32=not args.fp32)),
                         ("grad_x_pass", lambda: sinkhorn_geomloss_online_grad_sqeuclid(
                             x_dev, y_dev, a_w, b_w, torch.zeros(n, device=dev), gh + (y_dev**2).sum(1), eps=eps,
                             allow_tf32=not args.fp32, compute_grad_y=False)),
                         ("c_transform_pass", lambda: c_transform_fwd(x_dev, y_dev, gh, allow_tf32=not args.fp32))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record()
            for _ in range(5):
                fn()
            k1.record()
            torch.cuda.synchronize()
            res[name + "_ms"] = k0.elapsed_time(k1) / 5
            res[name + "_entries_per_s"] = n * m / (res[name + "_ms"] * 1e-3)
        print(json.dumps({"kernel_only": True, "n": n, "m": m, "d": d, "eps": eps,
                          "mode": "fp32(3xTF32)" if args.fp32 else "tf32", **res}))
        return 0

    def step_resident(x, y):
        xs = x.detach().requires_grad_(True)
        val = loss_fn(xs, y)
        (gx,) = torch.autograd.grad(val, xs)
        return val, gx

    def step_e2e():
        x = x_host.to(dev, non_blocking=True)
        y = y_host.to(dev, non_blocking=True)
        val, gx = step_resident(x, y)
        gx_host.copy_(gx, non_blocking=True)
        return float(val.item())  # device->host read of the loss closes the step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    x_dev, y_dev = x_host.to(dev), y_host.to(dev)
    for _ in range(args.warmup):
        step_resident(x_dev, y_dev)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = lib.fs_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        val, gx = step_resident(x_dev, y_dev)
    e1.record()
    barrier()
    launches = lib.fs_launch_count() - launches0
    ms = e0.elapsed_time(e1)
    # end-to-end: host buffers in, loss + gradient out
    step_e2e()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        loss_val = step_e2e()
    t1.record()
    barrier()
    ms_e2e = t0.elapsed_time(t1)
    clocks = sampler.stop()

    # dominant kernel (one soft-min pass over all n x m entries), timed alone on the launching stream
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse_fused
    gh = -(y_dev**2).sum(1)
    lb = torch.full((m,), -float(torch.log(torch.tensor(float(m)))), device=dev)
    for _ in range(3):
        flashsinkhorn_lse_fused(x_dev, y_dev, gh, lb, eps, allow_tf32=not args.fp32)
    reps = 10
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    k0.record()
    for _ in range(reps):
        flashsinkhorn_lse_fused(x_dev, y_dev, gh, lb, eps, allow_tf32=not args.fp32)
    k1.record()
    torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / reps

    # plan-times-matrix on a 50,000 x 64 N(0,1) matrix at the solved potentials (second item of the config)
    apply_ms = None
    if world == 1:
        from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle
        from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
        a_w = torch.full((n,), 1.0 / n, device=dev)
        b_w = torch.full((m,), 1.0 / m, device=dev)
        f_pot, g_pot = sinkhorn_flashstyle_symmetric(x_dev, y_dev, a_w, b_w, use_epsilon_scaling=False, eps=eps,
                                                     n_iters=iters, allow_tf32=not args.fp32)
        f_hat, g_hat = f_pot - (x_dev**2).sum(1), g_pot - (y_dev**2).sum(1)
        v_mat = torch.randn(m, d, generator=torch.Generator().manual_seed(7)).to(dev)
        for _ in range(3):
            apply_plan_mat_flashstyle(x_dev, y_dev, f_hat, g_hat, a_w.log(), b_w.log(), v_mat, eps=eps, axis=1,
                                      allow_tf32=not args.fp32)
        torch.cuda.synchronize()
        k0.record()
        for _ in range(reps):
            apply_plan_mat_flashstyle(x_dev, y_dev, f_hat, g_hat, a_w.log(), b_w.log(), v_mat, eps=eps, axis=1,
                                      allow_tf32=not args.fp32)
        k1.record()
        torch.cuda.synchronize()
        apply_ms = k0.elapsed_time(k1) / reps

    # The reference's own benchmark setting, timed directly: ONE OT(x, y) solve, no debiasing, no final
    # extrapolation = 101 Jacobi steps (2.5e9 * 202 entries); on N ranks the rows are sharded like the step.
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric as _solve
    aw = torch.full((n,), 1.0 / n, device=dev)
    bw = torch.full((m,), 1.0 / m, device=dev)

    def solve_once():
        return _solve(x_dev, y_dev, aw, bw, use_epsilon_scaling=False, eps=eps, n_iters=iters,
                      last_extrapolation=False, allow_tf32=not args.fp32, process_group=group)

    solve_once()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(3):
        solve_once()
    s1.record()
    barrier()
    ms_solve = s0.elapsed_time(s1) / 3
    # Host time to ENQUEUE one such solve (nothing inside it synchronises): Python loop, ctypes calls, tensor-map
    # encodes and NCCL launches. Next to the device time above it shows whether the host or the GPU binds.
    torch.cuda.synchronize()
    h0 = time.perf_counter()
    solve_once()
    host_enqueue_ms = (time.perf_counter() - h0) * 1e3
    barrier()

    times = torch.tensor([ms, ms_e2e, ms_solve], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_solve = times.tolist()

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        sm_mhz = clocks.get("sm_mhz") or 1965.0
        # exp roofline: ex2 issue rate MEASURED on this GPU by the library's micro-benchmark (all SMs, 32
        # warps/SM, register data only); nominal 16 ex2/clk/SM x 148 SMs x sampled clock kept for context.
        # tensor roofline: TF32 dense = half the measured bf16 rate, 2*d flops per entry (x3 in 3xTF32 mode)
        exp_nominal = 16 * 148 * sm_mhz * 1e6
        exp_measured = float(lib.fs_micro_exp_rate(0, 32))
        softmax_loop_rate = float(lib.fs_micro_exp_rate(1, 16))
        exp_peak = exp_measured if exp_measured > 0 else exp_nominal
        bf16 = peaks.get("bf16_tflops_sustained", 1400.0) * 1e12
        tc_peak = (bf16 / 2) / (2 * d * (3 if args.fp32 else 1))
        peak = min(exp_peak, tc_peak)
        achieved = n * m / (kernel_ms * 1e-3)
        total = per_step * args.steps  # strong scaling: the ranks share one problem
        line = {
            "metric": "cost_entries_per_sec", "value": total / (ms * 1e-3), "unit": "entries/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 (3xTF32 products)" if args.fp32 else "tf32 products, f32 accumulate/exp",
            "data": "synthetic",
            "config": {"workload": workload, "entries_per_step": per_step, "parallelism": (f"rows sharded over {world} GPUs, all-gather per half-step" if world > 1 else "single GPU"),
                       "l2": "inputs 25.6 MB < L2; the pass is "
                       "compute-bound (one exp + 2d flops per entry), L2 is not flushed between steps",
                       "self_terms": "OT(x,x), OT(y,y): one soft-min per step (f == g bit for bit)",
                       "ms_per_100iter_solve": ms_solve,
                       "ms_per_100iter_solve_note": "one OT(x,y) solve, debias off, last_extrapolation off "
                                                    f"({iters + 1} Jacobi steps), timed directly",
                       "host_enqueue_ms_per_100iter_solve": host_enqueue_ms,
                       "apply_plan_mat_ms": apply_ms,
                       # results of the last step, so that N-GPU and 1-GPU runs can be compared from the records
                       "loss": loss_val, "grad_x_abs_sum": float(gx.double().abs().sum().item()),
                       "grad_x_norm": float(gx.double().norm().item())},
            "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "entries/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": x_host.numel() * 4 + y_host.numel() * 4,
                    "d2h_bytes_per_step": gx_host.numel() * 4 + 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "exp" if exp_peak <= tc_peak else "tensor", "achieved": achieved, "peak": peak,
                         "unit": "entries/s", "frac": achieved / peak,
                         # DRAM bytes per launch of this kernel at this size, from an
                         # ncu capture of this kernel at this size (algorithmic: 29.2 MB of staged operands)
                         "traffic": 28925952 if (n == 50000 and m == 50000 and d == 64 and not args.fp32) else None,
                         "traffic_unit": "bytes per launch (dram read + write)",
                         "kernel": "row soft-min pass (fs_lse), n*m entries per launch", "kernel_ms": kernel_ms,
                         "exp_peak": exp_peak, "exp_peak_nominal": exp_nominal, "tensor_peak": tc_peak,
                         "softmax_loop_rate": softmax_loop_rate,
                         "peak_source": "of measured: ex2.approx rate from fs_micro_exp_rate(0,32) on this GPU; "
                                        "tensor = measured bf16 (MEASURED_PEAKS.json, sustained)/2 for TF32; "
                                        "nominal = 16 ex2/clk/SM x 148 SM x sampled SM clock"},
            "loss": loss_val,
        }
        if not args.skip_cpu and world == 1:
            cb, _, _ = cpu_reference_sample(n, m, d, eps)
            line["cpu_baseline"] = cb
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
