"""Autograd glue: OT cost with an analytic backward, and a gradient node whose backward is the HVP.

Behaviour follows the reference's ``_autograd.py`` (``_SinkhornConfig`` :33-76,
``_SinkhornGradFn`` :84-283, ``_SinkhornCostFn`` :291-519):

* forward = Sinkhorn solve + dual cost; the cost uses the final potentials, the
  gradient the potentials *before* the last extrapolation step (GeomLoss convention);
* ``d cost / d a = f``, ``d cost / d b = g`` (times the incoming gradient);
* ``d cost / d x`` comes from the barycentric gradient kernel and is itself
  differentiable w.r.t. x: its backward is the streaming-CG Hessian-vector product,
  always evaluated with fp32-exact products;
* double backward w.r.t. y raises ``NotImplementedError``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from flash_sinkhorn_b200.hvp import geomloss_to_ott_potentials, hvp_x_sqeuclid_from_potentials
from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid
from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating, sinkhorn_flashstyle_symmetric


@dataclass(frozen=True)
class _SinkhornConfig:
    """Immutable snapshot of a ``SamplesLoss`` configuration, carried on the autograd context."""

    backend: str
    blur: float
    scaling: float
    use_epsilon_scaling: bool
    eps: Optional[float]
    n_iters: Optional[int]
    cost_scale: float
    rho_x: Optional[float]
    rho_y: Optional[float]
    last_extrapolation: bool
    allow_tf32: bool
    use_exp2: bool
    autotune: bool
    block_m: Optional[int]
    block_n: Optional[int]
    block_k: Optional[int]
    num_warps: Optional[int]
    num_stages: int
    hvp_tau2: float
    hvp_max_cg_iter: int
    hvp_cg_rtol: float
    hvp_cg_atol: float
    hvp_cg_stabilise_every: int
    hvp_preconditioner: str
    hvp_precond_terms: int
    hvp_use_preconditioner: bool
    lambda_x: float
    lambda_y: float
    threshold: Optional[float]
    inner_iterations: int
    # Extension: torch.distributed group for row-sharded multi-GPU solves (None = single GPU).
    process_group: object = None


class _SinkhornGradFn(torch.autograd.Function):
    """``(grad_x, grad_y)`` of the OT cost; differentiable once more w.r.t. x (HVP)."""

    @staticmethod
    def forward(ctx, x, y, a, b, f_grad, g_grad, grad_scale, eps: float, config: _SinkhornConfig,
                want_x: bool, want_y: bool, label_x=None, label_y=None, label_cost_matrix=None):
        gx, gy = sinkhorn_geomloss_online_grad_sqeuclid(
            x, y, a, b, f_grad, g_grad,
            eps=float(eps), allow_tf32=config.allow_tf32, grad_scale=grad_scale,
            compute_grad_x=bool(want_x), compute_grad_y=bool(want_y), cost_scale=config.cost_scale,
            label_x=label_x, label_y=label_y, label_cost_matrix=label_cost_matrix,
            lambda_x=config.lambda_x, lambda_y=config.lambda_y,
            process_group=config.process_group,
        )
        ctx.save_for_backward(x, y, a, b, f_grad, g_grad, grad_scale)
        ctx.eps = float(eps)
        ctx.config = config
        ctx.use_label_cost = (label_x is not None and label_y is not None and label_cost_matrix is not None
                              and config.lambda_y != 0.0)
        return gx, gy

    @staticmethod
    def backward(ctx, v_x, v_y):
        x, y, a, b, f_grad, g_grad, grad_scale = ctx.saved_tensors
        cfg = ctx.config
        if v_y is not None:
            raise NotImplementedError("Double backward w.r.t y is not implemented yet.")
        if ctx.use_label_cost:
            raise NotImplementedError("Double backward (HVP) is not supported with OTDD label-augmented cost. "
                                      "Use gradient flow without HVP.")
        out_x = None
        if v_x is not None:
            if v_x.shape != x.shape:
                raise ValueError("grad_grad_x must have the same shape as x.")
            if not v_x.is_cuda:
                raise ValueError("grad_grad_x must be a CUDA tensor.")
            with torch.no_grad():
                f_ott, g_ott = geomloss_to_ott_potentials(f_grad, g_grad, a, b, eps=ctx.eps)
                hv, _ = hvp_x_sqeuclid_from_potentials(
                    x, y, f_ott, g_ott, v_x,
                    eps=ctx.eps, rho_x=cfg.rho_x, rho_y=cfg.rho_y, cost_scale=cfg.cost_scale,
                    tau2=cfg.hvp_tau2, max_cg_iter=cfg.hvp_max_cg_iter,
                    cg_rtol=cfg.hvp_cg_rtol, cg_atol=cfg.hvp_cg_atol,
                    cg_stabilise_every=cfg.hvp_cg_stabilise_every,
                    preconditioner=cfg.hvp_preconditioner, precond_terms=cfg.hvp_precond_terms,
                    use_preconditioner=cfg.hvp_use_preconditioner,
                    allow_tf32=False,  # second-order products need fp32-exact scores
                )
                out_x = hv * grad_scale
        return (out_x,) + (None,) * 13


class _SinkhornCostFn(torch.autograd.Function):
    """Entropic OT cost ``OT_eps(a, x; b, y)`` with an analytic (envelope-theorem) backward."""

    @staticmethod
    def forward(ctx, x, y, a, b, eps_list: Tuple[float, ...], config: _SinkhornConfig,
                label_x, label_y, label_cost_matrix, presolved=None):
        # `presolved` (extension): (f_cost, g_cost, f_grad, g_grad) from a solve done elsewhere - the multi-GPU
        # divergence solves its three problems interleaved before building the three cost nodes.
        label_kw = dict(label_x=label_x, label_y=label_y, label_cost_matrix=label_cost_matrix,
                        lambda_x=config.lambda_x, lambda_y=config.lambda_y)
        if presolved is not None:
            eps = float(eps_list[-1])
            f_cost, g_cost, f_grad, g_grad = presolved
            plain_dual = config.backend == "alternating" or config.rho_x is None or config.rho_y is None
        elif config.backend == "alternating":
            eps = float(eps_list[-1])
            f_cost, g_cost = sinkhorn_flashstyle_alternating(
                x, y, a, b, eps=eps, n_iters=len(eps_list), cost_scale=config.cost_scale,
                rho_x=config.rho_x, rho_y=config.rho_y, allow_tf32=config.allow_tf32,
                process_group=config.process_group,
            )
            f_grad, g_grad = f_cost, g_cost
            plain_dual = True  # the reference's alternating branch always returns <a,f>+<b,g>
        else:
            eps = float(eps_list[-1])
            common = dict(
                blur=config.blur, scaling=config.scaling, use_epsilon_scaling=config.use_epsilon_scaling,
                eps=config.eps, n_iters=config.n_iters, allow_tf32=config.allow_tf32,
                cost_scale=config.cost_scale, rho_x=config.rho_x, rho_y=config.rho_y,
                threshold=config.threshold, check_every=config.inner_iterations,
                process_group=config.process_group,
            )
            if config.last_extrapolation:
                f_cost, g_cost, f_grad, g_grad = sinkhorn_flashstyle_symmetric(
                    x, y, a, b, last_extrapolation=True, return_prelast=True, **common, **label_kw)
            else:
                f_cost, g_cost = sinkhorn_flashstyle_symmetric(x, y, a, b, last_extrapolation=False, **common,
                                                               **label_kw)
                f_grad, g_grad = f_cost, g_cost
            plain_dual = config.rho_x is None or config.rho_y is None  # balanced or semi-unbalanced

        ctx.save_for_backward(x, y, a, b, f_cost, g_cost, f_grad, g_grad)
        ctx.eps = eps
        ctx.config = config
        ctx.labels = (label_x, label_y, label_cost_matrix)

        if plain_dual:
            return (a * f_cost).sum() + (b * g_cost).sum()
        # Both marginals relaxed: (rho + eps/2) * <w, 1 - exp(-potential/rho)> per side.
        total = torch.tensor(0.0, device=x.device, dtype=torch.float32)
        total = total + (config.rho_x + eps / 2) * (a * (1 - (-f_cost / config.rho_x).exp())).sum()
        total = total + (config.rho_y + eps / 2) * (b * (1 - (-g_cost / config.rho_y).exp())).sum()
        return total

    @staticmethod
    def backward(ctx, grad_out):
        x, y, a, b, f_cost, g_cost, f_grad, g_grad = ctx.saved_tensors
        gx = gy = ga = gb = None
        if x.requires_grad or y.requires_grad:
            gx, gy = _SinkhornGradFn.apply(
                x, y, a, b, f_grad, g_grad, grad_out, ctx.eps, ctx.config, x.requires_grad, y.requires_grad,
                *ctx.labels)
            if not x.requires_grad:
                gx = None
            if not y.requires_grad:
                gy = None
        if a.requires_grad:
            ga = grad_out * f_cost
        if b.requires_grad:
            gb = grad_out * g_cost
        return gx, gy, ga, gb, None, None, None, None, None, None
