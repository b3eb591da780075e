"""Row-sharded (multi-GPU) Sinkhorn solves: one process per GPU, ``torch.distributed`` collectives.

The reference package is single-GPU. Here every rank holds the full clouds, weights and potentials
(they are O((n+m) d)); the n x m work of every step is split by rows: rank r produces rows
``[r*shard_f, (r+1)*shard_f)`` of the new f and the matching slice of the new g, then the slices are
all-gathered (two in-place all-gathers of n resp. m floats per step, NCCL over NVLink on GPUs).
Because every rank then holds identical full vectors, early-stop decisions are identical everywhere
without a further collective. Results equal the single-GPU engine's up to rounding: the kernels are the
same, but the streaming pass cuts its column range by the number of row blocks it is given, so the order
in which a row's partial sums are merged depends on the shard size.

The loops themselves (:func:`run_symmetric_sharded`, :func:`run_alternating_sharded`) are engine-agnostic -
they get the step and the gather as callables - so they are unit-tested on CPU with ``gloo`` and a dense
CPU step function. The alternating (Gauss-Seidel) solver shards the same way, with one all-gather after
every half-step.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

SHARD_ALIGN = 128  # rows; shards start on the kernels' 128-row half-block grid


def shard_layout(rows: int, world: int, align: int = SHARD_ALIGN) -> int:
    """Rows per rank (same on all ranks, multiple of ``align``; the last shards may be short or empty)."""
    per = -(-rows // world)
    return -(-per // align) * align


def shard_range(rows: int, world: int, rank: int, align: int = SHARD_ALIGN) -> Tuple[int, int]:
    shard = shard_layout(rows, world, align)
    return min(rows, rank * shard), min(rows, (rank + 1) * shard)


def balanced_tile_ranges(row_ptr, rows: int, world: int, tile: int = SHARD_ALIGN):
    """Row ranges ``[(lo, hi)] * world`` for a block-sparse pass: contiguous runs of ``tile``-row blocks whose
    numbers of kept tiles (CSR ``row_ptr`` over the row blocks, host values) are as equal as a cut at block
    boundaries allows. Rank r gets the blocks whose cumulative kept-tile count falls in the r-th of ``world``
    equal parts; empty ranges are possible when there are fewer blocks than ranks."""
    rp = [int(v) for v in row_ptr]
    nblk = len(rp) - 1
    total = rp[-1] - rp[0]
    cuts = [0]
    b = 0
    for r in range(1, world):
        target = rp[0] + (total * r) / world
        while b < nblk and (rp[b] + rp[b + 1]) / 2.0 < target:  # block goes to the side its middle lies on
            b += 1
        cuts.append(b)
    cuts.append(nblk)
    return [(min(rows, cuts[r] * tile), min(rows, cuts[r + 1] * tile)) for r in range(world)]


def sharded_steps(
    n: int,
    m: int,
    f_hat0: torch.Tensor,
    g_hat0: torch.Tensor,
    eps_list: Sequence[float],
    *,
    last_extrapolation: bool,
    threshold: Optional[float],
    check_every: int,
    world: int,
    rank: int,
    step_fn: Callable,
    gather_fn: Callable,
    self_problem: bool = False,
):
    """Generator form of the sharded symmetric schedule (init step, averaged loop, optional extrapolation).

    Yields after the launches of every step and finally returns the result tuple (``StopIteration.value``),
    so that a caller can interleave the steps of several independent problems: the gathers of one then
    overlap the compute of the next (see :func:`run_many`). :func:`run_symmetric_sharded` runs one problem.

    ``step_fn(f_old, g_old, f_new, g_new, eps, w, (f_lo, f_hi, g_lo, g_hi))`` must fill rows
    ``[f_lo, f_hi)`` of ``f_new`` and ``[g_lo, g_hi)`` of ``g_new`` from the full old potentials; it is
    called twice per step, first with an empty g range, then with an empty f range, so that the
    gather of the new f slices can overlap the g half (both halves read only OLD potentials).
    ``gather_fn(buf, shard)`` all-gathers ``buf`` in place (rank r owns ``buf[r*shard:(r+1)*shard]``)
    and may return a callable that waits for completion (asynchronous gather) or None.
    Buffers are padded to ``world*shard`` entries. Returns ``(f_hat, g_hat, f_hat_pre, g_hat_pre, steps)``.

    ``self_problem`` (same cloud, weights, penalties and initial potentials on both sides, ``n == m``):
    g equals f after every step, so only the f half runs (and is gathered) and g aliases f.
    """
    sf, sg = shard_layout(n, world), shard_layout(m, world)
    f_lo, f_hi = shard_range(n, world, rank)
    g_lo, g_hi = shard_range(m, world, rank)
    mk = lambda size, src: torch.zeros(size, dtype=src.dtype, device=src.device)
    f = [mk(world * sf, f_hat0), mk(world * sf, f_hat0)]
    f[0][:n].copy_(f_hat0)
    if self_problem:
        if n != m:
            raise ValueError("self_problem needs n == m")
        g = f
    else:
        g = [mk(world * sg, g_hat0), mk(world * sg, g_hat0)]
        g[0][:m].copy_(g_hat0)
    cur = 0
    pending = {"f": None, "g": None}  # waits for the (asynchronous) gathers that fill f[cur] / g[cur]
    parity = 0

    def settle(*sides):
        for sd in sides:
            if pending[sd] is not None:
                pending[sd]()
                pending[sd] = None

    def step(eps, w):
        # The half that produces new f needs the complete current g and vice versa. Alternating which
        # half goes first lets BOTH gathers hide behind a compute half: the gather launched last in one
        # step is only needed by the second half of the next step.
        nonlocal cur, parity
        if self_problem:
            settle("f")
            step_fn(f[cur], f[cur], f[cur ^ 1], f[cur ^ 1], float(eps), float(w), (f_lo, f_hi, g_lo, g_lo))
            pending["f"] = gather_fn(f[cur ^ 1], sf)
            cur ^= 1
            return
        launched = {}
        for side in (("f", "g") if parity == 0 else ("g", "f")):
            settle("g" if side == "f" else "f")
            rng = (f_lo, f_hi, g_lo, g_lo) if side == "f" else (f_lo, f_lo, g_lo, g_hi)
            step_fn(f[cur], g[cur], f[cur ^ 1], g[cur ^ 1], float(eps), float(w), rng)
            launched[side] = gather_fn(f[cur ^ 1], sf) if side == "f" else gather_fn(g[cur ^ 1], sg)
        settle("f", "g")  # nothing should be left; keeps the invariant obvious
        pending.update(launched)
        cur ^= 1
        parity ^= 1

    steps = 0
    step(eps_list[0], 1.0)
    steps += 1
    yield
    prev = None
    for i, eps in enumerate(eps_list):
        step(eps, 0.5)
        steps += 1
        yield
        if threshold is not None and (i + 1) % check_every == 0:
            settle("f", "g")
            if prev is None:
                prev = (f[cur][:n].clone(), g[cur][:m].clone())
            else:
                change = max(float((f[cur][:n] - prev[0]).abs().max()), float((g[cur][:m] - prev[1]).abs().max()))
                if change < threshold:  # identical on all ranks: the vectors are
                    break
                prev[0].copy_(f[cur][:n])
                prev[1].copy_(g[cur][:m])
    f_pre = g_pre = None
    if last_extrapolation:
        settle("f", "g")
        f_pre, g_pre = f[cur][:n].clone(), g[cur][:m].clone()
        step(eps_list[-1], 1.0)
        steps += 1
        yield
    settle("f", "g")
    return f[cur][:n].clone(), g[cur][:m].clone(), f_pre, g_pre, steps


def run_many(generators):
    """Round-robin over :func:`sharded_steps` generators until all are exhausted; results in input order."""
    gens = list(generators)
    results = [None] * len(gens)
    live = list(range(len(gens)))
    while live:
        for i in list(live):
            try:
                next(gens[i])
            except StopIteration as done:
                results[i] = done.value
                live.remove(i)
    return results


def run_symmetric_sharded(*args, **kwargs):
    """One problem through :func:`sharded_steps` (same arguments and result)."""
    return run_many([sharded_steps(*args, **kwargs)])[0]


class PackedLayout:
    """Where the potentials of several problems live in one buffer that a single all-gather completes.

    The buffer is ``[world, width]``: row r is what rank r produces in one step - for every problem its slice of
    f (``shard_f`` slots) and, unless the problem is a self-transport one, its slice of g. Element j of a full
    vector therefore sits at ``row j // shard``, column ``offset + j % shard``: the "packed" addressing that
    ``fs_symmetric_step_multi`` takes (shard size + row pitch), so that no copy sits between the kernel that
    writes the slices, the collective and the kernel that reads the full vectors."""

    def __init__(self, sizes, world: int):
        """``sizes`` = ``[(n, m, self_problem)]`` per problem."""
        self.world = world
        self.slots = []
        off = 0
        for n, m, self_problem in sizes:
            sf = shard_layout(n, world)
            f_slot = (off, sf, n)
            off += sf
            if self_problem:
                g_slot = f_slot
            else:
                sg = shard_layout(m, world)
                g_slot = (off, sg, m)
                off += sg
            self.slots.append((f_slot, g_slot))
        self.width = max(off, 1)

    def new_buffer(self, like: torch.Tensor) -> torch.Tensor:
        return torch.zeros(self.world * self.width, dtype=like.dtype, device=like.device)

    def full(self, buf: torch.Tensor, k: int, side: int) -> torch.Tensor:
        """Full vector of problem k (side 0 = f, 1 = g) gathered out of ``buf`` (a copy)."""
        off, shard, size = self.slots[k][side]
        return buf.view(self.world, self.width)[:, off:off + shard].reshape(-1)[:size].clone()

    def store(self, buf: torch.Tensor, k: int, side: int, vec: torch.Tensor) -> None:
        off, shard, size = self.slots[k][side]
        padded = torch.zeros(self.world * shard, dtype=buf.dtype, device=buf.device)
        padded[:size].copy_(vec)
        buf.view(self.world, self.width)[:, off:off + shard].copy_(padded.view(self.world, shard))


def run_symmetric_fused(problems, *, world: int, rank: int, step_fn: Callable, gather_fn: Callable):
    """Several symmetric solves in lockstep, every step of all of them as ONE fused launch and ONE all-gather.

    ``problems`` = list of dicts with ``n, m, f_hat0, g_hat0, eps_list, last_extrapolation, threshold,
    check_every, self_problem``. Step t of every problem that still has a step t is handed to
    ``step_fn(items, old_buf, new_buf, layout)`` at once; ``items`` = ``[(k, eps, w, (f_lo, f_hi, g_lo, g_hi))]``
    and the function must write rows ``[f_lo, f_hi)`` of problem k's new f (and ``[g_lo, g_hi)`` of its new g,
    unless the range is empty) into rank ``rank``'s row of ``new_buf`` at the layout's offsets, reading the full
    old vectors from ``old_buf``. ``gather_fn(buf, width)`` then completes ``new_buf`` in place. A problem that
    has finished keeps its slots unchanged (its values are carried over by a copy of its slots).
    Returns ``[(f_hat, g_hat, f_hat_pre, g_hat_pre, steps)]`` like :func:`sharded_steps`.
    """
    layout = PackedLayout([(p["n"], p["m"], p["self_problem"]) for p in problems], world)
    like = problems[0]["f_hat0"]
    buf = [layout.new_buffer(like), layout.new_buffer(like)]
    cur = 0
    plans, state = [], []
    for k, p in enumerate(problems):
        layout.store(buf[0], k, 0, p["f_hat0"])
        if not p["self_problem"]:
            layout.store(buf[0], k, 1, p["g_hat0"])
        eps = list(p["eps_list"])
        steps = [(eps[0], 1.0, "init")] + [(e, 0.5, "loop") for e in eps]
        if p["last_extrapolation"]:
            steps.append((eps[-1], 1.0, "last"))
        plans.append(steps)
        f_lo, f_hi = shard_range(p["n"], world, rank)
        g_lo, g_hi = shard_range(p["m"], world, rank)
        if p["self_problem"]:
            g_hi = g_lo  # only the f half runs; g aliases f
        state.append(dict(pos=0, done=False, rng=(f_lo, f_hi, g_lo, g_hi), prev=None, pre=(None, None), used=0,
                          loops=0))
    while True:
        items = []
        for k, (p, st) in enumerate(zip(problems, state)):
            if st["done"]:
                continue
            if st["pos"] >= len(plans[k]):
                st["done"] = True
                continue
            eps, w, kind = plans[k][st["pos"]]
            if kind == "last":  # the potentials before the final extrapolation are part of the result
                st["pre"] = (layout.full(buf[cur], k, 0), layout.full(buf[cur], k, 1))
            items.append((k, float(eps), float(w), st["rng"]))
        if not items:
            break
        active = {k for k, *_ in items}
        new = buf[cur ^ 1]
        for k in range(len(problems)):  # finished problems: carry their slots over unchanged
            if k not in active:
                for side in ((0,) if problems[k]["self_problem"] else (0, 1)):
                    off, shard, _ = layout.slots[k][side]
                    new.view(world, layout.width)[:, off:off + shard].copy_(
                        buf[cur].view(world, layout.width)[:, off:off + shard])
        step_fn(items, buf[cur], new, layout)
        wait = gather_fn(new, layout.width)
        if wait is not None:
            wait()
        cur ^= 1
        for k, eps, w, _ in items:
            p, st = problems[k], state[k]
            kind = plans[k][st["pos"]][2]
            st["pos"] += 1
            st["used"] += 1
            if kind != "loop":
                continue
            st["loops"] += 1
            if p["threshold"] is not None and st["loops"] % p["check_every"] == 0:
                f_now, g_now = layout.full(buf[cur], k, 0), layout.full(buf[cur], k, 1)
                if st["prev"] is not None:
                    change = max(float((f_now - st["prev"][0]).abs().max()), float((g_now - st["prev"][1]).abs().max()))
                    if change < p["threshold"]:  # identical on all ranks: the vectors are
                        st["pos"] = len(plans[k]) - 1 if p["last_extrapolation"] else len(plans[k])
                st["prev"] = (f_now, g_now)
    out = []
    for k, st in enumerate(state):
        out.append((layout.full(buf[cur], k, 0), layout.full(buf[cur], k, 1), st["pre"][0], st["pre"][1], st["used"]))
    return out


def _gather_inplace(group, overlap: bool = False):
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    side = torch.cuda.Stream() if overlap else None
    # a small ring of re-used events (a few gathers are in flight at any time, also with interleaved problems)
    events = [(torch.cuda.Event(), torch.cuda.Event()) for _ in range(16)] if overlap else []
    state = {"i": 0}

    def gather(buf: torch.Tensor, shard: int):
        if side is None:
            dist.all_gather_into_tensor(buf, buf[rank * shard:(rank + 1) * shard], group=group)
            return None
        # Run the collective on a side stream ordered after the kernels enqueued so far; the caller's
        # stream only waits for it when the returned callable is invoked.
        main = torch.cuda.current_stream()
        ready, done = events[state["i"] % len(events)]
        state["i"] += 1
        ready.record(main)
        side.wait_event(ready)
        with torch.cuda.stream(side):
            dist.all_gather_into_tensor(buf, buf[rank * shard:(rank + 1) * shard], group=group)
        done.record(side)
        return lambda: main.wait_event(done)

    return gather, world, rank


def _cuda_problem(x, y, log_a, log_b, eps_list, *, cost_scale, rho_x, rho_y, last_extrapolation,
                  threshold, check_every, f_init, g_init, prec, gather, world, rank):
    """(generator, finish) of one problem on the CUDA engine; ``finish(result)`` -> standard potentials."""
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels._common import dampening

    n, d = x.shape
    m = y.shape[0]
    dev = x.device
    alpha = cost_scale * x.pow(2).sum(dim=1)
    beta = cost_scale * y.pow(2).sum(dim=1)
    f0 = (f_init.float() - alpha) if f_init is not None else -alpha
    g0 = (g_init.float() - beta) if g_init is not None else -beta
    ws = _lib.workspace(_lib.OP_STEP, n, m, d, prec, dev)
    state = {"staged": False}

    def step_fn(f_old, g_old, f_new, g_new, eps, w, rng):
        df, dg = dampening(eps, rho_x), dampening(eps, rho_y)
        _lib.call(
            "fs_symmetric_step_range", dev,
            _lib.ptr(x), _lib.ptr(y), n, m, d, _lib.ptr(f_old), _lib.ptr(g_old), _lib.ptr(log_a), _lib.ptr(log_b),
            _lib.ptr(f_new), _lib.ptr(g_new), _lib.ptr(alpha), _lib.ptr(beta),
            eps, w, df, dg, float(cost_scale), rng[0], rng[1], rng[2], rng[3], 0 if state["staged"] else 1,
            prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
        )
        state["staged"] = True

    same_init = (f_init is None and g_init is None) or (
        f_init is not None and g_init is not None and f_init.data_ptr() == g_init.data_ptr())
    self_problem = (n == m and x.data_ptr() == y.data_ptr() and log_a.data_ptr() == log_b.data_ptr()
                    and same_init and rho_x == rho_y)
    gen = sharded_steps(
        n, m, f0, g0, eps_list, last_extrapolation=last_extrapolation, threshold=threshold,
        check_every=check_every, world=world, rank=rank, step_fn=step_fn, gather_fn=gather,
        self_problem=self_problem)

    def finish(result):
        fh, gh, fp, gp, steps = result
        out_pre = (None, None) if fp is None else (fp + alpha, gp + beta)
        return fh + alpha, gh + beta, out_pre[0], out_pre[1], steps

    return gen, finish


def _fused_solve_cuda(problems, group):
    """CUDA engine behind :func:`run_symmetric_fused`: one ``fs_symmetric_step_multi`` call and one all-gather per
    step for all problems together. Needs the tensor-core engine (the packed addressing of the potentials is
    read by its bias kernels); the caller checks ``fs_engine`` first."""
    import ctypes
    import os

    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels._common import dampening

    gather, world, rank = _gather_inplace(group)
    lib = _lib.load()
    dev = problems[0]["x"].device
    d = problems[0]["x"].shape[1]
    prec = problems[0]["prec"]
    prepared, consts = [], []
    for pr in problems:
        x, y = pr["x"], pr["y"]
        n, m = x.shape[0], y.shape[0]
        cs = pr["cost_scale"]
        alpha = cs * x.pow(2).sum(dim=1)
        beta = alpha if y.data_ptr() == x.data_ptr() and n == m else cs * y.pow(2).sum(dim=1)
        fi, gi = pr["f_init"], pr["g_init"]
        f0 = (fi.float() - alpha) if fi is not None else -alpha
        g0 = (gi.float() - beta) if gi is not None else -beta
        same_init = (fi is None and gi is None) or (fi is not None and gi is not None and fi.data_ptr() == gi.data_ptr())
        self_problem = (n == m and x.data_ptr() == y.data_ptr() and pr["log_a"].data_ptr() == pr["log_b"].data_ptr()
                        and same_init and pr["rho_x"] == pr["rho_y"])
        prepared.append(dict(n=n, m=m, f_hat0=f0, g_hat0=g0, eps_list=pr["eps_list"],
                             last_extrapolation=pr["last_extrapolation"], threshold=pr["threshold"],
                             check_every=pr["check_every"], self_problem=self_problem))
        consts.append(dict(alpha=alpha, beta=beta, ws=_lib.workspace(_lib.OP_STEP, n, m, d, prec, dev), staged=False))
    fsize = ctypes.sizeof(ctypes.c_float)

    def step_fn(items, old, new, layout):
        arr = (_lib.StepItem * len(items))()
        for slot, (k, eps, w, rng) in zip(arr, items):
            pr, c = problems[k], consts[k]
            (f_off, f_shard, _), (g_off, g_shard, _) = layout.slots[k]
            slot.x, slot.y, slot.n, slot.m = pr["x"].data_ptr(), pr["y"].data_ptr(), prepared[k]["n"], prepared[k]["m"]
            slot.f_hat, slot.g_hat = old.data_ptr() + fsize * f_off, old.data_ptr() + fsize * g_off
            slot.f_out, slot.g_out = new.data_ptr() + fsize * f_off, new.data_ptr() + fsize * g_off
            slot.log_a, slot.log_b = pr["log_a"].data_ptr(), pr["log_b"].data_ptr()
            slot.alpha_x, slot.beta_y = c["alpha"].data_ptr(), c["beta"].data_ptr()
            slot.eps, slot.w = eps, w
            slot.damp_f, slot.damp_g = dampening(eps, pr["rho_x"]), dampening(eps, pr["rho_y"])
            slot.cost_scale = pr["cost_scale"]
            slot.f_begin, slot.f_end, slot.g_begin, slot.g_end = rng
            slot.restage = 0 if c["staged"] else 1
            slot.ws, slot.ws_bytes = c["ws"].data_ptr(), c["ws"].numel()
            slot.f_shard, slot.g_shard, slot.pack_stride = f_shard, g_shard, layout.width
            c["staged"] = True
        _lib.call("fs_symmetric_step_multi", dev, ctypes.cast(arr, ctypes.c_void_p), len(items), d, prec,
                  _lib.stream_ptr(dev))

    results = run_symmetric_fused(prepared, world=world, rank=rank, step_fn=step_fn, gather_fn=gather)
    out = []
    for (fh, gh, fp, gp, steps), c in zip(results, consts):
        pre = (None, None) if fp is None else (fp + c["alpha"], gp + c["beta"])
        out.append((fh + c["alpha"], gh + c["beta"], pre[0], pre[1], steps))
    return out


def symmetric_solve_sharded_many(problems, *, group):
    """Solve several independent problems with their steps interleaved (each ``problems[i]`` is the keyword
    set of :func:`symmetric_solve_sharded` without ``group``). While one problem's all-gather is in flight
    the next problem computes, which hides the exchange even for self-transport problems, whose single
    half-step per iteration leaves nothing of their own to overlap with."""
    import os

    from flash_sinkhorn_b200 import _lib

    # Tensor-core shapes: every step of all problems as one fused launch + one all-gather (the fixed cost of a
    # launch is then paid once per step instead of once per pass, which is what a short per-rank pass needs).
    # FLASH_SINKHORN_B200_FUSED_STEPS=0 keeps the pass-by-pass schedule below (overlapped gathers).
    d = problems[0]["x"].shape[1]
    same = all(pr["x"].shape[1] == d and pr["prec"] == problems[0]["prec"] for pr in problems)
    tc_engine = all(_lib.load().fs_engine(pr["x"].shape[0], pr["y"].shape[0], d, pr["prec"]) >= 1 for pr in problems)
    if same and tc_engine and len(problems) <= 8 and os.environ.get("FLASH_SINKHORN_B200_FUSED_STEPS", "1") != "0":
        return _fused_solve_cuda(problems, group)
    gather, world, rank = _gather_inplace(group, overlap=True)
    built = [_cuda_problem(gather=gather, world=world, rank=rank, **pr) for pr in problems]
    # The all-gather of one half-step runs next to the streaming pass of the next one; that pass is a single
    # wave of one CTA per SM, so it leaves a few SMs to the collective instead of waiting for them.
    lib = _lib.load()
    previous = lib.fs_set_reserved_sms(int(os.environ.get("FLASH_SINKHORN_B200_RESERVED_SMS", "2")))
    try:
        results = run_many([g for g, _ in built])
    finally:
        lib.fs_set_reserved_sms(previous)
    return [fin(res) for (_, fin), res in zip(built, results)]


def symmetric_solve_sharded(x, y, log_a, log_b, eps_list, *, group, **kw):
    """CUDA engine behind :func:`run_symmetric_sharded`. Returns standard potentials like the 1-GPU solver."""
    return symmetric_solve_sharded_many([dict(x=x, y=y, log_a=log_a, log_b=log_b, eps_list=eps_list, **kw)],
                                        group=group)[0]


def run_alternating_sharded(
    n: int,
    m: int,
    f_hat0: torch.Tensor,
    g_hat0: torch.Tensor,
    eps_list: Sequence[float],
    iters_per_eps: int,
    *,
    ott_convention: bool,
    threshold: Optional[float],
    check_every: int,
    world: int,
    rank: int,
    half_fn: Callable,
    gather_fn: Callable,
    ranges: Optional[dict] = None,
):
    """Row-sharded Gauss-Seidel (alternating) schedule: every half-step needs the COMPLETE result of the
    previous one, so each is followed by its all-gather before the next starts (nothing to overlap inside
    one problem; the n x m work of each half is still split ``world`` ways).

    ``half_fn(side, f_cur, g_cur, out, eps, (lo, hi))`` must fill rows ``[lo, hi)`` of ``out`` with the new
    potential of ``side`` ("f": from ``g_cur``; "g": from ``f_cur``), ``out`` never aliasing the inputs.
    GeomLoss convention runs f then g, the OTT convention g then f (reference sinkhorn_solvers.py:188-259).
    ``eps_list`` x ``iters_per_eps`` is the annealed form (one stage = the reference's fixed-eps loop).
    Early stop as in the reference (:264-270): every ``check_every`` iterations, against the potentials of
    the previous check (the initial ones at first); identical on all ranks since the vectors are.
    ``ranges`` (optional) = ``{"f": [(lo, hi)] * world, "g": [...]}``: explicit, possibly unequal row ranges per
    rank (block-sparse passes are split by kept tiles, see :func:`balanced_tile_ranges`). The gather then goes
    through a padded staging buffer with one equal-sized slot per rank.
    Returns ``(f_hat, g_hat, iterations)``.
    """
    if ranges is not None:
        return _run_alternating_ranges(n, m, f_hat0, g_hat0, eps_list, iters_per_eps, ott_convention=ott_convention,
                                       threshold=threshold, check_every=check_every, world=world, rank=rank,
                                       half_fn=half_fn, gather_fn=gather_fn, ranges=ranges)
    sf, sg = shard_layout(n, world), shard_layout(m, world)
    rows = {"f": shard_range(n, world, rank), "g": shard_range(m, world, rank)}
    mk = lambda size, src: torch.zeros(size, dtype=src.dtype, device=src.device)
    buf = {"f": [mk(world * sf, f_hat0), mk(world * sf, f_hat0)], "g": [mk(world * sg, g_hat0), mk(world * sg, g_hat0)]}
    buf["f"][0][:n].copy_(f_hat0)
    buf["g"][0][:m].copy_(g_hat0)
    cur = {"f": 0, "g": 0}
    shard = {"f": sf, "g": sg}
    order = ("g", "f") if ott_convention else ("f", "g")

    def half(side, eps):
        out = buf[side][cur[side] ^ 1]
        half_fn(side, buf["f"][cur["f"]], buf["g"][cur["g"]], out, float(eps), rows[side])
        wait = gather_fn(out, shard[side])
        if wait is not None:
            wait()
        cur[side] ^= 1

    prev = (f_hat0.clone(), g_hat0.clone())
    used = 0
    stop = False
    for eps in eps_list:
        for _ in range(int(iters_per_eps)):
            for side in order:
                half(side, eps)
            used += 1
            if threshold is not None and used % check_every == 0:
                f_now, g_now = buf["f"][cur["f"]][:n], buf["g"][cur["g"]][:m]
                change = max(float((f_now - prev[0]).abs().max()), float((g_now - prev[1]).abs().max()))
                if change < threshold:
                    stop = True
                    break
                prev[0].copy_(f_now)
                prev[1].copy_(g_now)
        if stop:
            break
    return buf["f"][cur["f"]][:n].clone(), buf["g"][cur["g"]][:m].clone(), used


def _run_alternating_ranges(n, m, f_hat0, g_hat0, eps_list, iters_per_eps, *, ott_convention, threshold,
                            check_every, world, rank, half_fn, gather_fn, ranges):
    """:func:`run_alternating_sharded` with explicit row ranges per rank. Rank r writes its rows into slot r of
    a ``[world, longest range]`` staging buffer, the slots are all-gathered, and every rank copies each slot
    back to its rows of the full vector."""
    size = {"f": n, "g": m}
    full = {"f": [f_hat0.clone(), f_hat0.clone()], "g": [g_hat0.clone(), g_hat0.clone()]}
    cur = {"f": 0, "g": 0}
    slot = {sd: max(1, max(hi - lo for lo, hi in ranges[sd])) for sd in ("f", "g")}
    stage = {sd: torch.zeros(world * slot[sd], dtype=f_hat0.dtype, device=f_hat0.device) for sd in ("f", "g")}
    order = ("g", "f") if ott_convention else ("f", "g")

    def half(side, eps):
        out = full[side][cur[side] ^ 1]
        lo, hi = ranges[side][rank]
        half_fn(side, full["f"][cur["f"]], full["g"][cur["g"]], out, float(eps), (lo, hi))
        if hi > lo:
            stage[side][rank * slot[side]: rank * slot[side] + (hi - lo)].copy_(out[lo:hi])
        wait = gather_fn(stage[side], slot[side])
        if wait is not None:
            wait()
        for r, (rlo, rhi) in enumerate(ranges[side]):
            if rhi > rlo and r != rank:
                out[rlo:rhi].copy_(stage[side][r * slot[side]: r * slot[side] + (rhi - rlo)])
        cur[side] ^= 1

    prev = (f_hat0.clone(), g_hat0.clone())
    used = 0
    stop = False
    for eps in eps_list:
        for _ in range(int(iters_per_eps)):
            for side in order:
                half(side, eps)
            used += 1
            if threshold is not None and used % check_every == 0:
                f_now, g_now = full["f"][cur["f"]][:size["f"]], full["g"][cur["g"]][:size["g"]]
                change = max(float((f_now - prev[0]).abs().max()), float((g_now - prev[1]).abs().max()))
                if change < threshold:
                    stop = True
                    break
                prev[0].copy_(f_now)
                prev[1].copy_(g_now)
        if stop:
            break
    return full["f"][cur["f"]].clone(), full["g"][cur["g"]].clone(), used


def alternating_solve_sharded(x, y, log_a, log_b, eps_list, iters_per_eps, *, cost_scale, rho_x, rho_y,
                              ott_convention, threshold, check_every, prec, group, tile_csr=None,
                              tile_row_counts=None):
    """CUDA engine behind :func:`run_alternating_sharded`: a half-step is ``fs_symmetric_step_range`` with
    weight 1, one empty row range and no shift correction (the alternating solver has none). In the OTT
    convention the log-weights stay out of the soft-min and ``eps*log w`` is added to the produced rows.
    ``tile_csr`` = the four device CSR arrays of a block-sparse tile list and of its transpose (as
    ``fs_solve_alternating`` takes them) and ``tile_row_counts`` = ``(row_ptr, row_ptr_t)`` as host sequences:
    the rows of every half-step are then split so that each rank gets about the same number of kept tiles.
    Returns standard potentials ``(f, g, iterations)`` like the 1-GPU solver."""
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels._common import dampening

    n, d = x.shape
    m = y.shape[0]
    dev = x.device
    gather, world, rank = _gather_inplace(group)
    alpha = cost_scale * x.pow(2).sum(dim=1)
    beta = cost_scale * y.pow(2).sum(dim=1)
    ws = _lib.workspace(_lib.OP_STEP, n, m, d, prec, dev)
    ranges = None
    csr = (None, None, None, None)
    if tile_csr is not None:
        csr = tuple(tile_csr)
        ranges = {"f": balanced_tile_ranges(tile_row_counts[0], n, world),
                  "g": balanced_tile_ranges(tile_row_counts[1], m, world)}
    zeros_a, zeros_b = torch.zeros_like(log_a), torch.zeros_like(log_b)
    in_a, in_b = (zeros_a, zeros_b) if ott_convention else (log_a, log_b)
    # the entry point wants an output for both sides; the side with the empty range is never written
    spare = {"f": torch.empty(n, device=dev, dtype=torch.float32), "g": torch.empty(m, device=dev, dtype=torch.float32)}
    state = {"staged": False}

    def half_fn(side, f_cur, g_cur, out, eps, rng):
        lo, hi = rng
        f_out, g_out = (out, spare["g"]) if side == "f" else (spare["f"], out)
        rr = (lo, hi, 0, 0) if side == "f" else (0, 0, lo, hi)
        _lib.call(
            "fs_symmetric_step_range_tiles", dev,
            _lib.ptr(x), _lib.ptr(y), n, m, d, _lib.ptr(f_cur), _lib.ptr(g_cur), _lib.ptr(in_a), _lib.ptr(in_b),
            _lib.ptr(f_out), _lib.ptr(g_out), None, None,
            eps, 1.0, dampening(eps, rho_x), dampening(eps, rho_y), float(cost_scale),
            rr[0], rr[1], rr[2], rr[3], 0 if state["staged"] else 1,
            _lib.ptr(csr[0]), _lib.ptr(csr[1]), _lib.ptr(csr[2]), _lib.ptr(csr[3]),
            prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
        )
        state["staged"] = True
        if ott_convention and hi > lo:
            out[lo:hi].add_((log_a if side == "f" else log_b)[lo:hi], alpha=eps)

    fh, gh, used = run_alternating_sharded(
        n, m, -alpha, -beta, eps_list, iters_per_eps, ott_convention=ott_convention, threshold=threshold,
        check_every=check_every, world=world, rank=rank, half_fn=half_fn, gather_fn=gather, ranges=ranges)
    return fh + alpha, gh + beta, used


def grad_sharded(x, y, a, b, log_a, log_b, f, g, grad_scale, eps, cost_scale, prec, want_x, want_y, group):
    """Row-sharded analytic gradient: each rank computes its rows, slices are all-gathered."""
    from flash_sinkhorn_b200 import _lib

    n, d = x.shape
    m = y.shape[0]
    dev = x.device
    gather, world, rank = _gather_inplace(group)
    sx, sy = shard_layout(n, world), shard_layout(m, world)
    x_lo, x_hi = shard_range(n, world, rank)
    y_lo, y_hi = shard_range(m, world, rank)
    gx = torch.zeros((world * sx, d), device=dev, dtype=torch.float32) if want_x else None
    gy = torch.zeros((world * sy, d), device=dev, dtype=torch.float32) if want_y else None
    ws = _lib.workspace(_lib.OP_GRAD, n, m, d, prec, dev)
    _lib.call(
        "fs_grad_range", dev,
        _lib.ptr(x), _lib.ptr(y), n, m, d, _lib.ptr(a), _lib.ptr(b), _lib.ptr(log_a), _lib.ptr(log_b),
        _lib.ptr(f), _lib.ptr(g), _lib.ptr(grad_scale), _lib.ptr(gx), _lib.ptr(gy),
        float(eps), float(cost_scale), x_lo, x_hi, y_lo, y_hi, prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    if want_x:
        gather(gx.view(-1), sx * d)
        gx = gx[:n]
    if want_y:
        gather(gy.view(-1), sy * d)
        gy = gy[:m]
    return gx, gy
