"""``SamplesLoss``: GeomLoss-style front end of the B200 Sinkhorn engine.

Drop-in for the reference's ``samples_loss.py`` (argument parsing :73-191, constructor
:260-414, eps schedule :451-470, forward :472-597): same constructor keywords and
defaults, the two call forms ``loss(x, y)`` / ``loss(a, x, b, y)``, ``(N, D)`` or batched
``(B, N, D)`` clouds, the same ValueError / TypeError / DeprecationWarning behaviour.
Triton tuning keywords are stored and ignored. The OTDD label-augmented cost
(``label_cost_matrix``, ``lambda_x``, ``lambda_y``; labels given to ``forward``) is supported on the
symmetric backend for forward and gradient; its double backward raises ``NotImplementedError`` as in
the reference.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple, Union

import torch

from flash_sinkhorn_b200._autograd import _SinkhornConfig, _SinkhornCostFn
from flash_sinkhorn_b200.kernels._common import epsilon_schedule, max_diameter
from flash_sinkhorn_b200.sinkhorn_solvers import (
    sinkhorn_flashstyle_symmetric_batched,
    sinkhorn_flashstyle_alternating,
    sinkhorn_flashstyle_symmetric,
    sinkhorn_flashstyle_symmetric_many,
)


@dataclass(frozen=True)
class _ParsedInputs:
    x: torch.Tensor
    y: torch.Tensor
    a: torch.Tensor
    b: torch.Tensor
    batched: bool
    a_view_shape: Tuple[int, ...]
    b_view_shape: Tuple[int, ...]


def _as_float_tensor(t) -> torch.Tensor:
    if not torch.is_tensor(t):
        raise TypeError("Expected a torch.Tensor.")
    if not t.is_floating_point():
        raise TypeError("Expected a floating-point tensor.")
    return t


def _normalize_weights(w: torch.Tensor, *, eps: float = 0.0) -> torch.Tensor:
    """Weights divided by their sum along the last axis (sum clamped at 1e-40)."""
    w = w.float()
    if eps > 0:
        w = w + eps
    return w / w.sum(dim=-1, keepdim=True).clamp(min=1e-40)


def _weights_for(w, pts: torch.Tensor, lead: Tuple[int, ...], count: int, name: str, cloud: str):
    """Default to uniform weights, accept a trailing singleton axis, reject anything else."""
    flat = lead + (count,)
    if w is None:
        return torch.full(flat, 1.0 / count, device=pts.device, dtype=torch.float32), flat
    w = _as_float_tensor(w)
    if tuple(w.shape) == flat:
        return w, flat
    if tuple(w.shape) == flat + (1,):
        return w[..., 0], flat + (1,)
    if lead:
        letter = "n" if name == "a" else "m"
        raise ValueError(f"{name} must have shape (B,{letter}) or (B,{letter},1) matching {cloud}.")
    letter = "n" if name == "a" else "m"
    raise ValueError(f"{name} must have shape ({letter},) or ({letter},1) matching {cloud}.")


def _process_args(*args, normalize: bool) -> _ParsedInputs:
    if len(args) == 2:
        (x, y), a, b = args, None, None
    elif len(args) == 4:
        a, x, b, y = args
    else:
        raise TypeError(f"SamplesLoss expects either (x, y) or (a, x, b, y). Got {len(args)} arguments.")
    x, y = _as_float_tensor(x), _as_float_tensor(y)

    if x.ndim == 2:
        lead: Tuple[int, ...] = ()
        (n, dx), (m, dy) = x.shape, y.shape
    elif x.ndim == 3:
        if y.ndim != 3:
            raise ValueError("If x is batched (B,N,D), y must be batched too.")
        (bx, n, dx), (by, m, dy) = x.shape, y.shape
        if bx != by:
            raise ValueError("x and y must have the same batch size.")
        lead = (bx,)
    else:
        raise ValueError("x and y must be shaped (N,D) or (B,N,D).")
    if dx != dy:
        raise ValueError("x and y must have the same feature dimension.")

    a, a_shape = _weights_for(a, x, lead, n, "a", "x")
    b, b_shape = _weights_for(b, y, lead, m, "b", "y")
    if normalize:
        a, b = _normalize_weights(a), _normalize_weights(b)
    return _ParsedInputs(x, y, a, b, bool(lead), a_shape, b_shape)


class SamplesLoss(torch.nn.Module):
    """Entropic OT loss between weighted point clouds (squared Euclidean ground cost, CUDA only).

    * ``loss`` must be ``"sinkhorn"`` and ``p`` must be 2.
    * ``blur`` sets the final temperature ``eps = blur**2``; with ``use_epsilon_scaling`` the
      solver anneals from the clouds' diameter with ratio ``scaling**2`` (``n_iters`` then only
      truncates that schedule); otherwise give a fixed ``eps`` and ``n_iters``.
    * ``reach`` / ``reach_x`` / ``reach_y`` relax the marginals (``rho = reach**2``); ``reach``
      fills whichever side was not given.
    * ``debias`` returns ``OT(a,b) - OT(a,a)/2 - OT(b,b)/2``.
    * ``half_cost`` uses ``|x-y|^2/2``.
    * ``backend="symmetric"`` (default, Jacobi averaged steps) or ``"alternating"``
      (Gauss-Seidel; needs fixed ``eps`` and ``n_iters``).
    * ``threshold`` / ``inner_iterations`` enable early stopping, checked every
      ``inner_iterations`` steps on the device.
    * ``potentials=True`` returns ``(f, g)`` (no autograd) instead of the cost.

    The cost is differentiable w.r.t. x, y (analytic gradient at the pre-extrapolation
    potentials), a, b, and twice w.r.t. x (Hessian-vector products via streaming CG, tuned by
    the ``hvp_*`` keywords).
    """

    def __init__(
        self,
        loss: str = "sinkhorn",
        *,
        p: int = 2,
        blur: float = 0.05,
        reach: Optional[float] = None,
        reach_x: Optional[float] = None,
        reach_y: Optional[float] = None,
        scaling: float = 0.5,
        debias: bool = False,
        potentials: bool = False,
        backend: str = "symmetric",
        normalize: bool = True,
        use_epsilon_scaling: bool = True,
        last_extrapolation: bool = True,
        allow_tf32: bool = True,
        use_exp2: bool = True,
        autotune: bool = True,
        half_cost: bool = False,
        eps: Optional[float] = None,
        n_iters: Optional[int] = None,
        diameter: Optional[float] = None,
        eps_list: Optional[Sequence[float]] = None,
        block_m: Optional[int] = None,
        block_n: Optional[int] = None,
        block_k: Optional[int] = None,
        num_warps: Optional[int] = None,
        num_stages: int = 2,
        hvp_tau2: float = 1e-5,
        hvp_max_cg_iter: int = 300,
        hvp_cg_rtol: float = 1e-6,
        hvp_cg_atol: float = 1e-6,
        hvp_cg_stabilise_every: int = 0,
        hvp_preconditioner: str = "none",
        hvp_precond_terms: int = 3,
        hvp_use_preconditioner: bool = True,
        label_cost_matrix: Optional[torch.Tensor] = None,
        lambda_x: float = 1.0,
        lambda_y: float = 0.0,
        threshold: Optional[float] = None,
        inner_iterations: int = 10,
        use_flashstyle: Optional[bool] = None,
        process_group=None,
    ):
        super().__init__()
        if use_flashstyle is not None and not use_flashstyle:
            warnings.warn(
                "use_flashstyle=False is deprecated. FlashSinkhorn is now the only backend.",
                DeprecationWarning, stacklevel=2,
            )
        if loss != "sinkhorn":
            raise ValueError('Only loss="sinkhorn" is supported.')
        if p != 2:
            raise ValueError("Only p=2 (squared Euclidean cost) is supported.")
        if backend not in ("symmetric", "alternating", "triton", "auto"):
            raise ValueError('Only backend in {"symmetric","alternating","triton","auto"} is supported.')
        if backend in ("triton", "auto"):
            warnings.warn(
                f'backend="{backend}" is a legacy alias for "symmetric". '
                'Use backend="symmetric" or backend="alternating" explicitly.',
                DeprecationWarning, stacklevel=2,
            )
            backend = "symmetric"
        if backend == "alternating":
            if use_epsilon_scaling:
                raise ValueError('backend="alternating" requires use_epsilon_scaling=False. '
                                 "Provide fixed eps and n_iters instead.")
            if eps is None or n_iters is None:
                raise ValueError('backend="alternating" requires eps and n_iters to be specified.')
            if label_cost_matrix is not None:
                raise ValueError('backend="alternating" does not support OTDD label cost. '
                                 'Use backend="symmetric" for label-augmented cost.')
        for name, val, what in (("reach", reach, "OT"), ("reach_x", reach_x, "source"), ("reach_y", reach_y, "target")):
            if val is not None and val <= 0:
                raise ValueError(f"{name} must be positive (or None for balanced {what}).")
        if reach is not None:
            reach_x = reach if reach_x is None else reach_x
            reach_y = reach if reach_y is None else reach_y

        self.loss, self.p = loss, p
        self.blur = float(blur)
        self.reach_x = None if reach_x is None else float(reach_x)
        self.reach_y = None if reach_y is None else float(reach_y)
        self.rho_x = None if reach_x is None else float(reach_x) ** 2
        self.rho_y = None if reach_y is None else float(reach_y) ** 2
        same = reach_x == reach_y
        self.reach = self.reach_x if same else None
        self.rho = self.rho_x if same else None
        self.scaling = float(scaling)
        self.debias, self.potentials = bool(debias), bool(potentials)
        self.backend, self.normalize = backend, bool(normalize)
        self.use_epsilon_scaling = bool(use_epsilon_scaling)
        self.last_extrapolation = bool(last_extrapolation)
        self.allow_tf32, self.use_exp2, self.autotune = bool(allow_tf32), bool(use_exp2), bool(autotune)
        self.half_cost = bool(half_cost)
        self.cost_scale = 0.5 if half_cost else 1.0
        self.eps = None if eps is None else float(eps)
        self.n_iters = None if n_iters is None else int(n_iters)
        self.diameter = None if diameter is None else float(diameter)
        self.eps_list = None if eps_list is None else [float(e) for e in eps_list]
        self.block_m, self.block_n, self.block_k = block_m, block_n, block_k
        self.num_warps, self.num_stages = num_warps, int(num_stages)
        self.hvp_tau2 = float(hvp_tau2)
        self.hvp_max_cg_iter = int(hvp_max_cg_iter)
        self.hvp_cg_rtol, self.hvp_cg_atol = float(hvp_cg_rtol), float(hvp_cg_atol)
        self.hvp_cg_stabilise_every = int(hvp_cg_stabilise_every)
        self.hvp_preconditioner = str(hvp_preconditioner)
        self.hvp_precond_terms = int(hvp_precond_terms)
        self.hvp_use_preconditioner = bool(hvp_use_preconditioner)
        self.label_cost_matrix = label_cost_matrix
        self.lambda_x, self.lambda_y = float(lambda_x), float(lambda_y)
        self.threshold = None if threshold is None else float(threshold)
        self.inner_iterations = int(inner_iterations)
        # Extension (no reference counterpart): torch.distributed group, one rank per GPU; the symmetric
        # solver and the gradient shard their rows over it. Every rank must call with the same inputs.
        self.process_group = process_group

    def _make_config(self) -> _SinkhornConfig:
        return _SinkhornConfig(
            backend=self.backend, blur=self.blur, scaling=self.scaling,
            use_epsilon_scaling=self.use_epsilon_scaling, eps=self.eps, n_iters=self.n_iters,
            cost_scale=self.cost_scale, rho_x=self.rho_x, rho_y=self.rho_y,
            last_extrapolation=self.last_extrapolation, allow_tf32=self.allow_tf32, use_exp2=self.use_exp2,
            autotune=self.autotune, block_m=self.block_m, block_n=self.block_n, block_k=self.block_k,
            num_warps=self.num_warps, num_stages=self.num_stages, hvp_tau2=self.hvp_tau2,
            hvp_max_cg_iter=self.hvp_max_cg_iter, hvp_cg_rtol=self.hvp_cg_rtol, hvp_cg_atol=self.hvp_cg_atol,
            hvp_cg_stabilise_every=self.hvp_cg_stabilise_every, hvp_preconditioner=self.hvp_preconditioner,
            hvp_precond_terms=self.hvp_precond_terms, hvp_use_preconditioner=self.hvp_use_preconditioner,
            lambda_x=self.lambda_x, lambda_y=self.lambda_y, threshold=self.threshold,
            inner_iterations=self.inner_iterations, process_group=self.process_group,
        )

    def _eps_list_for_inputs(self, x: torch.Tensor, y: torch.Tensor) -> Sequence[float]:
        """Schedule whose last entry is the eps the gradient / HVP / unbalanced cost use.

        As in the reference, the symmetric solver rebuilds its own schedule from
        blur/scaling/eps/n_iters; ``eps_list`` and ``diameter`` given to the constructor
        only reach this list.
        """
        if self.eps_list is not None:
            sched = list(self.eps_list)
        elif self.use_epsilon_scaling:
            diam = self.diameter if self.diameter is not None else max_diameter(x, y)
            sched = list(epsilon_schedule(diam, self.blur, self.scaling, p=2.0))
        else:
            if self.eps is None or self.n_iters is None:
                raise ValueError("When use_epsilon_scaling=False, provide eps and n_iters.")
            sched = [float(self.eps)] * int(self.n_iters)
        if self.n_iters is not None:
            sched = sched[: int(self.n_iters)]
        if not sched:
            raise ValueError("eps_list is empty after applying n_iters.")
        return sched

    def _symmetric_potentials(self, x, y, a, b, label_x, label_y):
        return sinkhorn_flashstyle_symmetric(
            x, y, a, b, blur=self.blur, scaling=self.scaling, use_epsilon_scaling=self.use_epsilon_scaling,
            eps=self.eps, n_iters=self.n_iters, allow_tf32=self.allow_tf32, cost_scale=self.cost_scale,
            rho_x=self.rho_x, rho_y=self.rho_y, last_extrapolation=self.last_extrapolation,
            label_x=label_x, label_y=label_y, label_cost_matrix=self.label_cost_matrix,
            lambda_x=self.lambda_x, lambda_y=self.lambda_y,
            threshold=self.threshold, check_every=self.inner_iterations, process_group=self.process_group,
        )

    def forward(self, *args, label_x: Optional[torch.Tensor] = None, label_y: Optional[torch.Tensor] = None):
        parsed = _process_args(*args, normalize=self.normalize)
        if not parsed.x.is_cuda or not parsed.y.is_cuda:
            raise ValueError("flash_sinkhorn.SamplesLoss requires CUDA tensors.")
        config = self._make_config()

        def ot(xs, ys, ws_a, ws_b, lx, ly, presolved=None):
            sched = tuple(self._eps_list_for_inputs(xs, ys))
            return _SinkhornCostFn.apply(xs, ys, ws_a, ws_b, sched, config, lx, ly, self.label_cost_matrix,
                                         presolved)

        multi_gpu = (self.process_group is not None and self.backend != "alternating"
                     and torch.distributed.get_world_size(self.process_group) > 1)

        def divergence(xs, ys, ws_a, ws_b):
            if not self.debias:
                return ot(xs, ys, ws_a, ws_b, label_x, label_y)
            terms = [(xs, ys, ws_a, ws_b, label_x, label_y), (xs, xs, ws_a, ws_a, label_x, label_x),
                     (ys, ys, ws_b, ws_b, label_y, label_y)]
            pre = [None, None, None]
            if multi_gpu and self.label_cost_matrix is not None and label_x is not None and self.lambda_y != 0.0:
                raise NotImplementedError("The label cost is not available in the multi-GPU sharded solver.")
            if multi_gpu:
                # The three solves are independent: run them interleaved so that the all-gather of one
                # overlaps the compute of the next, then hand the potentials to the cost nodes.
                with torch.no_grad():
                    sols = sinkhorn_flashstyle_symmetric_many(
                        [(t[0].detach(), t[1].detach(), t[2].detach(), t[3].detach()) for t in terms],
                        process_group=self.process_group, blur=self.blur, scaling=self.scaling,
                        use_epsilon_scaling=self.use_epsilon_scaling, eps=self.eps, n_iters=self.n_iters,
                        allow_tf32=self.allow_tf32, cost_scale=self.cost_scale, rho_x=self.rho_x,
                        rho_y=self.rho_y, last_extrapolation=self.last_extrapolation,
                        threshold=self.threshold, check_every=self.inner_iterations)
                pre = [(f, g, f, g) if fp is None else (f, g, fp, gp) for (f, g, fp, gp, _) in sols]
            cross, self_x, self_y = (ot(*t, presolved=p) for t, p in zip(terms, pre))
            return cross - 0.5 * self_x - 0.5 * self_y

        # Batched inputs: the reference loops over the items (samples_loss.py:515-552). Here all symmetric solves of
        # the batch - three per item for the debiased loss - go to the library in ONE call and advance in lockstep,
        # several soft-min passes per launch; the cost / gradient nodes then receive the finished potentials. Early
        # stopping, the label cost, the alternating backend and sharded runs keep the per-item loop.
        labels_on = (self.label_cost_matrix is not None and label_x is not None and label_y is not None
                     and self.lambda_y != 0.0)
        if (parsed.batched and self.backend != "alternating" and self.threshold is None and not labels_on
                and not multi_gpu):
            items = list(zip(parsed.x, parsed.y, parsed.a, parsed.b))
            groups = []
            for xs, ys, wa, wb in items:
                if self.debias and not self.potentials:
                    groups.append([(xs, ys, wa, wb), (xs, xs, wa, wa), (ys, ys, wb, wb)])
                else:
                    groups.append([(xs, ys, wa, wb)])
            # detached views keep their storage, which is how the solver recognises a self-transport problem
            flat = [tuple(t.detach() for t in prob) for grp in groups for prob in grp]
            with torch.no_grad():
                sols = sinkhorn_flashstyle_symmetric_batched(
                    flat, blur=self.blur, scaling=self.scaling, use_epsilon_scaling=self.use_epsilon_scaling,
                    eps=self.eps, n_iters=self.n_iters, allow_tf32=self.allow_tf32, cost_scale=self.cost_scale,
                    rho_x=self.rho_x, rho_y=self.rho_y, last_extrapolation=self.last_extrapolation)
            if self.potentials:
                f = torch.stack([sol[0] for sol in sols], dim=0).view(parsed.a_view_shape)
                g = torch.stack([sol[1] for sol in sols], dim=0).view(parsed.b_view_shape)
                return f, g
            vals, k = [], 0
            for grp in groups:
                terms = [ot(*prob, label_x, label_y, presolved=sols[k + j][:4]) for j, prob in enumerate(grp)]
                k += len(grp)
                vals.append(terms[0] - 0.5 * terms[1] - 0.5 * terms[2] if len(terms) == 3 else terms[0])
            return torch.stack(vals, dim=0)

        if parsed.batched:
            items = zip(parsed.x, parsed.y, parsed.a, parsed.b)
            if self.potentials:
                pairs = [self._symmetric_potentials(xs, ys, wa, wb, label_x, label_y) for xs, ys, wa, wb in items]
                f = torch.stack([p[0] for p in pairs], dim=0).view(parsed.a_view_shape)
                g = torch.stack([p[1] for p in pairs], dim=0).view(parsed.b_view_shape)
                return f, g
            return torch.stack([divergence(xs, ys, wa, wb) for xs, ys, wa, wb in items], dim=0)

        if self.potentials:
            sched = self._eps_list_for_inputs(parsed.x, parsed.y)
            if self.backend == "alternating":
                f, g = sinkhorn_flashstyle_alternating(
                    parsed.x, parsed.y, parsed.a, parsed.b, eps=float(sched[-1]), n_iters=len(sched),
                    cost_scale=self.cost_scale, reach_x=self.reach_x, reach_y=self.reach_y,
                    allow_tf32=self.allow_tf32, process_group=self.process_group,
                )
            else:
                f, g = self._symmetric_potentials(parsed.x, parsed.y, parsed.a, parsed.b, label_x, label_y)
            return f.view(parsed.a_view_shape), g.view(parsed.b_view_shape)

        return divergence(parsed.x, parsed.y, parsed.a, parsed.b)
