"""Sinkhorn solver entry points (symmetric / alternating) over the CUDA engine.

Signatures, defaults, return shapes and error behaviour follow the reference's
``sinkhorn_solvers.py`` (sinkhorn_flashstyle_alternating :30-287,
sinkhorn_flashstyle_symmetric :290-707). Unlike the reference, the iteration loop
itself runs inside the library (``fs_solve_symmetric`` / ``fs_solve_alternating``):
the eps schedule, damping, shift correction, Jacobi averaging and the early-stop test
are enqueued on the current stream without any host synchronisation. The only sync
is the optional read-back of the iteration counter (``return_n_iters=True``).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from flash_sinkhorn_b200 import _lib
from flash_sinkhorn_b200.kernels._common import (
    epsilon_schedule,
    log_weights,
    max_diameter,
    resolve_marginal_penalties,
)

__all__ = ["sinkhorn_flashstyle_alternating", "sinkhorn_flashstyle_symmetric", "sinkhorn_flashstyle_symmetric_batched",
           "tile_mask_to_csr"]


def _same_tensor(u: Optional[torch.Tensor], v: Optional[torch.Tensor]) -> bool:
    """True when u and v are the same view of the same memory (identity, or e.g. two ``detach()`` of one tensor)."""
    if u is v:
        return True
    if u is None or v is None:
        return False
    return (u.data_ptr() == v.data_ptr() and u.shape == v.shape and u.stride() == v.stride()
            and u.dtype == v.dtype and u.device == v.device)


def _neg_if_none(v: Optional[float]) -> float:
    return -1.0 if v is None else float(v)


def _eps_array(eps_list: Sequence[float]):
    arr = (ctypes.c_double * len(eps_list))(*[float(e) for e in eps_list])
    return arr


_CSR_CACHE: dict = {}


def tile_mask_to_csr(mask: torch.Tensor, device: torch.device):
    """Boolean ``[ceil(n/128), ceil(m/128)]`` tile mask -> CSR arrays of the mask and of its transpose.

    Returns ``(row_ptr, col_idx, row_ptr_t, col_idx_t)`` as int32 device tensors, the form
    ``fs_solve_alternating`` takes for block-sparse tile skipping.
    """
    if mask.ndim != 2:
        raise ValueError("tile mask must be 2D")
    # The conversion walks the whole mask on the host (61M tiles at n = m = 1e6); a solve that is repeated with
    # the same, unmodified mask tensor re-uses the arrays of the previous call.
    key = (mask.data_ptr(), mask._version, tuple(mask.shape), str(mask.device), str(device))
    if _CSR_CACHE.get("key") == key:
        return _CSR_CACHE["csr"]
    mk = mask.to(device="cpu", dtype=torch.bool)

    def one(mt: torch.Tensor):
        counts = mt.sum(dim=1)
        rp = torch.zeros(mt.shape[0] + 1, dtype=torch.int64)
        rp[1:] = torch.cumsum(counts, dim=0)
        ci = mt.nonzero(as_tuple=False)[:, 1]
        return rp.to(torch.int32).to(device), ci.to(torch.int32).to(device).contiguous()

    rp, ci = one(mk)
    rpt, cit = one(mk.t().contiguous())
    _CSR_CACHE.update(key=key, csr=(rp, ci, rpt, cit), mask=mask,  # holding the mask keeps its address from being re-used
                      counts=([0] + torch.cumsum(mk.sum(dim=1), dim=0).tolist(),
                              [0] + torch.cumsum(mk.sum(dim=0), dim=0).tolist()))
    return rp, ci, rpt, cit


def sinkhorn_flashstyle_alternating(
    x: torch.Tensor,
    y: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    eps: float = 0.1,
    n_iters: int = 100,
    cost_scale: float = 1.0,
    rho: Optional[float] = None,
    reach: Optional[float] = None,
    rho_x: Optional[float] = None,
    rho_y: Optional[float] = None,
    reach_x: Optional[float] = None,
    reach_y: Optional[float] = None,
    allow_tf32: bool = True,
    use_exp2: bool = True,
    autotune: bool = True,
    threshold: Optional[float] = None,
    check_every: int = 5,
    return_n_iters: bool = False,
    ott_convention: bool = False,
    eps_list: Optional[Sequence[float]] = None,
    iters_per_eps: Optional[int] = None,
    tile_mask: Optional[torch.Tensor] = None,
    process_group=None,
):
    """Gauss-Seidel Sinkhorn at fixed ``eps``: f from g, then g from the new f.

    Returns ``(f, g)`` (plus the iteration count with ``return_n_iters``). In the default
    GeomLoss convention the log-weights sit inside the soft-min; ``ott_convention=True``
    updates g first and keeps ``eps*log a``, ``eps*log b`` outside. Damped (unbalanced)
    updates get no shift correction, exactly like the reference.

    Extensions without a reference counterpart: ``eps_list`` + ``iters_per_eps`` run an
    annealed sequence of fixed-eps stages, each warm-started from the previous one, and
    ``tile_mask`` (bool ``[ceil(n/128), ceil(m/128)]``) drops 128x128 tiles from both soft-mins.
    ``process_group``: a ``torch.distributed`` group with one rank per GPU and the same inputs on every
    rank; the rows of every half-step are split over the ranks and all-gathered
    (:func:`flash_sinkhorn_b200.distributed.alternating_solve_sharded`); with ``tile_mask`` the split is by kept
    tiles, so that every rank gets the same share of the work whatever the sparsity pattern.
    """
    n, d = x.shape
    m = y.shape[0]
    rho_x, rho_y = resolve_marginal_penalties(rho, reach, rho_x, rho_y, reach_x, reach_y)
    dev = _lib.require_cuda(x=x, y=y, a=a, b=b)

    if eps_list is None:
        stages, per_stage = [float(eps)], int(n_iters)
    else:
        stages = [float(e) for e in eps_list]
        per_stage = int(n_iters if iters_per_eps is None else iters_per_eps)
        if len(stages) == 0:
            raise ValueError("eps_list must be non-empty")

    x32, y32 = _lib.f32c(x), _lib.f32c(y)
    log_a, log_b = log_weights(a).contiguous(), log_weights(b).contiguous()
    prec = _lib.precision_id(allow_tf32)
    csr = (None, None, None, None)
    if tile_mask is not None:
        nt, mt = (n + 127) // 128, (m + 127) // 128
        if tuple(tile_mask.shape) != (nt, mt):
            raise ValueError(f"tile_mask must have shape ({nt}, {mt})")
        csr = tile_mask_to_csr(tile_mask, dev)
    if process_group is not None and torch.distributed.get_world_size(process_group) > 1:
        from flash_sinkhorn_b200.distributed import alternating_solve_sharded

        tiles = {}
        if tile_mask is not None:  # rows are then split by kept tiles, not by row count
            tiles = dict(tile_csr=csr, tile_row_counts=_CSR_CACHE["counts"])
        f, g, used = alternating_solve_sharded(
            x32, y32, log_a.float(), log_b.float(), stages, per_stage, cost_scale=float(cost_scale), rho_x=rho_x,
            rho_y=rho_y, ott_convention=bool(ott_convention), threshold=threshold, check_every=int(check_every),
            prec=prec, group=process_group, **tiles)
        return (f, g, used) if return_n_iters else (f, g)
    f = torch.empty((n,), device=dev, dtype=torch.float32)
    g = torch.empty((m,), device=dev, dtype=torch.float32)
    iters = torch.zeros((1,), device=dev, dtype=torch.int32)
    ws = _lib.workspace(_lib.OP_SOLVE_ALTERNATING, n, m, d, prec, dev)
    eps_arr = _eps_array(stages)
    _lib.call(
        "fs_solve_alternating", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d, _lib.ptr(log_a), _lib.ptr(log_b),
        ctypes.cast(eps_arr, ctypes.c_void_p), len(stages), per_stage,
        float(cost_scale), _neg_if_none(rho_x), _neg_if_none(rho_y),
        1 if ott_convention else 0, _neg_if_none(threshold), int(check_every),
        _lib.ptr(csr[0]), _lib.ptr(csr[1]), _lib.ptr(csr[2]), _lib.ptr(csr[3]),
        _lib.ptr(f), _lib.ptr(g), _lib.ptr(iters),
        prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev),
    )
    if return_n_iters:
        used = int(iters.item())
        _lib.raise_if_device_timeout(dev)  # the host has synchronised anyway: surface a device-side time-out
        return f, g, used
    return f, g


def sinkhorn_flashstyle_symmetric(
    x: torch.Tensor,
    y: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    blur: float = 0.05,
    scaling: float = 0.5,
    use_epsilon_scaling: bool = True,
    last_extrapolation: bool = True,
    cost_scale: float = 1.0,
    eps: Optional[float] = None,
    n_iters: Optional[int] = None,
    diameter: Optional[float] = None,
    eps_list: Optional[Sequence[float]] = None,
    rho: Optional[float] = None,
    reach: Optional[float] = None,
    rho_x: Optional[float] = None,
    rho_y: Optional[float] = None,
    reach_x: Optional[float] = None,
    reach_y: Optional[float] = None,
    allow_tf32: bool = True,
    use_exp2: bool = True,
    autotune: bool = True,
    fused: Optional[bool] = None,
    threshold: Optional[float] = None,
    check_every: int = 5,
    return_n_iters: bool = False,
    return_prelast: bool = False,
    f_init: Optional[torch.Tensor] = None,
    g_init: Optional[torch.Tensor] = None,
    label_x: Optional[torch.Tensor] = None,
    label_y: Optional[torch.Tensor] = None,
    label_cost_matrix: Optional[torch.Tensor] = None,
    lambda_x: float = 1.0,
    lambda_y: float = 0.0,
    process_group=None,
    _prepare_only: bool = False,
):
    """GeomLoss-style symmetric Sinkhorn (Jacobi steps averaged with weight 1/2).

    ``process_group`` (extension, no reference counterpart): a ``torch.distributed`` group with one
    rank per GPU. Every rank passes the same full inputs; the rows of each step are sharded over
    the ranks and all-gathered (see :mod:`flash_sinkhorn_b200.distributed`). Results are identical
    on all ranks.


    Step sequence: one full step at ``eps_list[0]``, one averaged step per schedule entry,
    and (``last_extrapolation``) one full step at the last eps. Returns standard potentials
    ``(f, g)``; with ``return_prelast`` (and extrapolation on) also the potentials before the
    last step, and with ``return_n_iters`` the number of steps taken. ``fused`` is accepted
    and ignored (one implementation serves both of the reference's paths).
    """
    n, d = x.shape
    m = y.shape[0]
    # OTDD label-augmented cost (reference sinkhorn_solvers.py:323-328, :557-560): the table lookup rides in
    # the tensor-core contraction as 3V extra operand columns, so no kernel differs from the plain solve.
    labels = _lib.LabelCost.make(label_x, label_y, label_cost_matrix, lambda_x, lambda_y, n, m, x.device)
    if labels is not None and fused is False:
        raise ValueError("OTDD label cost requires fused=True (default). Set fused=True or omit label_cost_matrix.")
    multi_gpu = process_group is not None and torch.distributed.get_world_size(process_group) > 1
    if labels is not None and multi_gpu:
        raise NotImplementedError("The label cost is not available in the multi-GPU sharded solver.")
    rho_x, rho_y = resolve_marginal_penalties(rho, reach, rho_x, rho_y, reach_x, reach_y)

    if eps_list is None:
        if use_epsilon_scaling:
            if diameter is None:
                diameter = max_diameter(x, y)
            eps_list = epsilon_schedule(diameter, blur, scaling, p=2.0)
        else:
            if eps is None or n_iters is None:
                raise ValueError("When use_epsilon_scaling=False, provide eps and n_iters")
            eps_list = [float(eps)] * int(n_iters)
    if len(eps_list) == 0:
        raise ValueError("eps_list must be non-empty")
    if n_iters is not None:
        eps_list = list(eps_list)[: int(n_iters)]
    if len(eps_list) == 0:
        raise ValueError("eps_list must be non-empty")

    dev = _lib.require_cuda(x=x, y=y, a=a, b=b, f_init=f_init, g_init=g_init)
    # A self-transport problem (OT(a,a): the debiasing terms pass the same tensors twice) keeps the same
    # buffers on both sides; the engine recognises it by pointer equality and runs one soft-min per step.
    x32 = _lib.f32c(x)
    y32 = x32 if _same_tensor(y, x) else _lib.f32c(y)
    log_a = log_weights(a).contiguous()
    log_b = log_a if _same_tensor(b, a) else log_weights(b).contiguous()
    fi = None if f_init is None else _lib.f32c(f_init)
    gi = None if g_init is None else (fi if _same_tensor(g_init, f_init) else _lib.f32c(g_init))
    prec = _lib.precision_id(allow_tf32)

    if multi_gpu:
        from flash_sinkhorn_b200.distributed import symmetric_solve_sharded

        sharded_args = dict(
            x=x32, y=y32, log_a=log_a, log_b=log_b, eps_list=list(eps_list), cost_scale=float(cost_scale),
            rho_x=rho_x, rho_y=rho_y, last_extrapolation=bool(last_extrapolation), threshold=threshold,
            check_every=int(check_every), f_init=fi, g_init=gi, prec=prec)
        if _prepare_only:
            return sharded_args
        f, g, f_pre, g_pre, steps = symmetric_solve_sharded(group=process_group, **sharded_args)
        out = (f, g)
        if return_prelast and last_extrapolation:
            out = out + (f_pre, g_pre)
        if return_n_iters:
            out = out + (int(steps),)
        return out

    f = torch.empty((n,), device=dev, dtype=torch.float32)
    g = torch.empty((m,), device=dev, dtype=torch.float32)
    want_pre = bool(return_prelast and last_extrapolation)
    f_pre = torch.empty((n,), device=dev, dtype=torch.float32) if want_pre else None
    g_pre = torch.empty((m,), device=dev, dtype=torch.float32) if want_pre else None
    iters = torch.zeros((1,), device=dev, dtype=torch.int32) if return_n_iters else None
    ws = _lib.workspace(_lib.OP_SOLVE_SYMMETRIC, n, m, d, prec, dev, labels.V if labels else 0)
    eps_arr = _eps_array(eps_list)
    _lib.call(
        "fs_solve_symmetric", dev,
        _lib.ptr(x32), _lib.ptr(y32), n, m, d, _lib.ptr(log_a), _lib.ptr(log_b),
        ctypes.cast(eps_arr, ctypes.c_void_p), len(eps_list), 1 if last_extrapolation else 0,
        float(cost_scale), _neg_if_none(rho_x), _neg_if_none(rho_y),
        _neg_if_none(threshold), int(check_every),
        _lib.ptr(fi), _lib.ptr(gi), _lib.ptr(f), _lib.ptr(g), _lib.ptr(f_pre), _lib.ptr(g_pre),
        _lib.ptr(iters),
        prec, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev), labels.ref if labels else None,
    )
    out = (f, g)
    if want_pre:
        out = out + (f_pre, g_pre)
    if return_n_iters:
        out = out + (int(iters.item()),)
        _lib.raise_if_device_timeout(dev)  # the host has synchronised anyway: surface a device-side time-out
    return out


def sinkhorn_flashstyle_symmetric_batched(
    problems,
    *,
    blur: float = 0.05,
    scaling: float = 0.5,
    use_epsilon_scaling: bool = True,
    last_extrapolation: bool = True,
    cost_scale: float = 1.0,
    eps: Optional[float] = None,
    n_iters: Optional[int] = None,
    rho: Optional[float] = None,
    reach: Optional[float] = None,
    rho_x: Optional[float] = None,
    rho_y: Optional[float] = None,
    reach_x: Optional[float] = None,
    reach_y: Optional[float] = None,
    allow_tf32: bool = True,
):
    """Several independent symmetric solves in ONE library call (``fs_solve_symmetric_batched``).

    Extension without a reference counterpart (the reference loops over batch items in Python,
    samples_loss.py:515-552). ``problems`` is a sequence of ``(x, y, a, b)`` with one feature dimension; every
    problem gets the schedule :func:`sinkhorn_flashstyle_symmetric` would give it (its own diameter with
    ``use_epsilon_scaling``), and all of them advance in lockstep, up to four soft-min passes per kernel launch.
    No early stopping, warm start or label cost. Returns one ``(f, g, f_prelast, g_prelast, n_steps)`` per problem
    (the pre-extrapolation pair equals ``(f, g)`` without ``last_extrapolation``); results equal the one-at-a-time
    solves up to the merge order of partial sums (rounding level). A problem given as ``(x, x, a, a)`` - the same
    tensors twice - is solved as a self-transport problem with one soft-min per step.
    """
    rho_x, rho_y = resolve_marginal_penalties(rho, reach, rho_x, rho_y, reach_x, reach_y)
    problems = list(problems)
    if not problems:
        return []
    d = problems[0][0].shape[1]
    prec = _lib.precision_id(allow_tf32)
    arr = (_lib.BatchItem * len(problems))()
    keep, outs = [], []
    dev = None
    for slot, (x, y, a, b) in zip(arr, problems):
        if x.shape[1] != d or y.shape[1] != d:
            raise ValueError("all problems of a batched solve must share the feature dimension")
        pdev = _lib.require_cuda(x=x, y=y, a=a, b=b)
        if dev is None:
            dev = pdev
        elif pdev != dev:
            raise ValueError("all problems of a batched solve must be on the same device")
        n, m = x.shape[0], y.shape[0]
        if use_epsilon_scaling:
            sched = epsilon_schedule(max_diameter(x, y), blur, scaling, p=2.0)
        else:
            if eps is None or n_iters is None:
                raise ValueError("When use_epsilon_scaling=False, provide eps and n_iters")
            sched = [float(eps)] * int(n_iters)
        if n_iters is not None:
            sched = list(sched)[: int(n_iters)]
        if len(sched) == 0:
            raise ValueError("eps_list must be non-empty")
        x32 = _lib.f32c(x)
        y32 = x32 if _same_tensor(y, x) else _lib.f32c(y)
        la = log_weights(a).contiguous()
        lb = la if _same_tensor(b, a) else log_weights(b).contiguous()
        f = torch.empty((n,), device=dev, dtype=torch.float32)
        g = torch.empty((m,), device=dev, dtype=torch.float32)
        fp = torch.empty((n,), device=dev, dtype=torch.float32)
        gp = torch.empty((m,), device=dev, dtype=torch.float32)
        ws = _lib.workspace(_lib.OP_SOLVE_SYMMETRIC, n, m, d, prec, dev)
        eps_arr = _eps_array(sched)
        keep += [x32, y32, la, lb, ws, eps_arr]
        slot.x, slot.y, slot.n, slot.m = x32.data_ptr(), y32.data_ptr(), n, m
        slot.log_a, slot.log_b = la.data_ptr(), lb.data_ptr()
        slot.eps_list_host, slot.n_eps = ctypes.cast(eps_arr, ctypes.c_void_p), len(sched)
        slot.f, slot.g, slot.f_pre, slot.g_pre = f.data_ptr(), g.data_ptr(), fp.data_ptr(), gp.data_ptr()
        slot.ws, slot.ws_bytes = ws.data_ptr(), ws.numel()
        outs.append((f, g, fp, gp, len(sched) + 1 + (1 if last_extrapolation else 0)))
    _lib.call("fs_solve_symmetric_batched", dev, ctypes.cast(arr, ctypes.c_void_p), len(problems), d,
              1 if last_extrapolation else 0, float(cost_scale), _neg_if_none(rho_x), _neg_if_none(rho_y), prec,
              _lib.stream_ptr(dev))
    return outs


def sinkhorn_flashstyle_symmetric_many(problems, *, process_group, **kwargs):
    """Several independent symmetric solves on a multi-GPU ``process_group`` with their steps interleaved.

    Extension without a reference counterpart. ``problems`` is a sequence of ``(x, y, a, b)``; ``kwargs``
    are keyword arguments of :func:`sinkhorn_flashstyle_symmetric` shared by all of them. Returns one
    ``(f, g, f_prelast, g_prelast, n_steps)`` tuple per problem (the pre-extrapolation potentials are
    ``None`` without ``last_extrapolation``). Each result equals the one-at-a-time solve bit for bit;
    interleaving only lets the all-gather of one problem overlap the compute of the next.
    """
    from flash_sinkhorn_b200.distributed import symmetric_solve_sharded_many

    if process_group is None or torch.distributed.get_world_size(process_group) < 2:
        raise ValueError("sinkhorn_flashstyle_symmetric_many needs a process group with at least two ranks")
    for drop in ("return_n_iters", "return_prelast", "_prepare_only"):
        kwargs.pop(drop, None)
    prepared = [
        sinkhorn_flashstyle_symmetric(x, y, a, b, process_group=process_group, _prepare_only=True, **kwargs)
        for (x, y, a, b) in problems
    ]
    return symmetric_solve_sharded_many(prepared, group=process_group)
