"""K-streamed tensor-core passes (feature dimensions whose operands do not fit in shared memory) and block-sparse
tile lists on the tensor cores, against dense fp64 on the same inputs.

The reference switches to a separate tiled kernel for large d (kernels/sinkhorn_triton_grad_sqeuclid.py:406-791,
switch at :962-1000) and tests it for d in {1025, 2048, 4096} (testing/test_geomloss_sinkhorn_triton.py:255-322);
here every streaming entry point is checked at such shapes. Tolerances: 2e-4 in the exact (3xTF32) mode; in TF32
mode the engine solves the exact problem for the TF32-rounded points, so it is compared with fp64 on inputs
rounded the same way (round-to-nearest onto 10 mantissa bits) - 2e-3 on soft-mins, plan-times-vector and
gradients, 1e-2 on plan-times-matrix (weights and matrix are rounded to TF32 once more for the second product).
"""
import math
import os

import numpy as np
import pytest
import torch

from gpu_util import dev, host, rel

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _tf32(t):
    i = t.contiguous().view(torch.int32)
    return ((i + 0x1000) & ~0x1FFF).view(torch.float32)


def _r(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


SHAPES = [(700, 900, 300), (700, 900, 128), (600, 1100, 2048), (257, 130, 515), (1, 300, 1025), (300, 1, 260),
          (400, 500, 230), (130, 3000, 90)]


@pytest.mark.parametrize("tf32", [False, True])
@pytest.mark.parametrize("n,m,d", SHAPES)
def test_streamed_passes_vs_dense_fp64(n, m, d, tf32):
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
    from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse
    g = torch.Generator().manual_seed(n + m + d)
    x = (torch.randn(n, d, generator=g) / d**0.5).cuda()
    y = (torch.randn(m, d, generator=g) / d**0.5 + 0.1).cuda()
    bias = torch.randn(m, generator=g).cuda()
    eps = 0.05
    t_lse, t_vec, t_mat = (2e-3, 2e-3, 1e-2) if tf32 else (2e-4, 2e-4, 2e-4)
    xr, yr = (_tf32(x), _tf32(y)) if tf32 else (x, y)
    dot = xr.double() @ yr.double().T
    want = -eps * torch.logsumexp((2.0 / eps) * dot + bias.double()[None], dim=1)
    got = flashsinkhorn_lse(x, y, bias, eps, allow_tf32=tf32)
    assert _r(got, want) < t_lse
    assert torch.equal(got, flashsinkhorn_lse(x, y, bias, eps, allow_tf32=tf32))  # run-to-run identical bits
    # a consistent pair of potentials: f_hat is the soft-min of g_hat, so P has row sums a
    a = torch.softmax(torch.randn(n, generator=g), 0).cuda()
    b = torch.softmax(torch.randn(m, generator=g), 0).cuda()
    la, lb = a.log(), b.log()
    gh = -(y**2).sum(1) + 0.01 * torch.randn(m, generator=g).cuda()
    fh = flashsinkhorn_lse(x, y, gh / eps + lb, eps, allow_tf32=False)
    S = (2 * dot + fh.double()[:, None] + gh.double()[None]) / eps + la.double()[:, None] + lb.double()[None]
    P = S.exp()
    v, u = torch.randn(m, generator=g).cuda(), torch.randn(n, generator=g).cuda()
    kw = dict(eps=eps, allow_tf32=tf32)
    assert _r(apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, v, axis=1, **kw), P @ v.double()) < t_vec
    assert _r(apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, u, axis=0, **kw), P.T @ u.double()) < t_vec
    V, U = torch.randn(m, d, generator=g).cuda(), torch.randn(n, d, generator=g).cuda()
    sc = torch.rand(m, generator=g).cuda()
    assert _r(apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, V, axis=1, scale=sc, **kw),
              P @ (V.double() * sc.double()[:, None])) < t_mat
    assert _r(apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, U, axis=0, **kw), P.T @ U.double()) < t_mat
    f, gp = fh + (x**2).sum(1), gh + (y**2).sum(1)
    gx, gy = sinkhorn_geomloss_online_grad_sqeuclid(x, y, a, b, f, gp, eps=eps, allow_tf32=tf32)
    Wx = torch.softmax(S - la.double()[:, None], dim=1)
    Wy = torch.softmax((S - lb.double()[None]).T, dim=1)
    assert _r(gx, 2 * a.double()[:, None] * (xr.double() - Wx @ yr.double())) < t_vec
    assert _r(gy, 2 * b.double()[:, None] * (yr.double() - Wy @ xr.double())) < t_vec
    assert _lib.load().fs_device_error() == 0


def test_large_d_solver_and_loss_match_the_cuda_core_engine(monkeypatch):
    """Semi-unbalanced SamplesLoss at d = 1100 (forward, grad_x): the K-streamed tensor-core path in exact mode
    against the CUDA-core fp32 engine on the same inputs (the engines share no kernel)."""
    from flash_sinkhorn_b200 import SamplesLoss
    g = torch.Generator().manual_seed(11)
    n, m, d = 500, 640, 1100
    x = torch.nn.functional.normalize(torch.randn(n, d, generator=g), dim=1).cuda()
    y = torch.nn.functional.normalize(torch.randn(m, d, generator=g), dim=1).cuda()
    out = {}
    for mode in ("simt", "fp32", "tf32"):
        monkeypatch.setenv("FLASH_SINKHORN_B200_PREC", mode)
        xs = x.clone().requires_grad_(True)
        val = SamplesLoss("sinkhorn", blur=0.2, reach_x=1.0, half_cost=True, use_epsilon_scaling=False, eps=0.04,
                          n_iters=20, allow_tf32=(mode == "tf32"))(xs, y)
        (gx,) = torch.autograd.grad(val, xs)
        out[mode] = (float(val), gx)
    assert abs(out["fp32"][0] - out["simt"][0]) <= 2e-5 * abs(out["simt"][0])
    assert _r(out["fp32"][1], out["simt"][1]) < 3e-4
    assert abs(out["tf32"][0] - out["simt"][0]) <= 1e-4 * abs(out["simt"][0])
    assert _r(out["tf32"][1], out["simt"][1]) < 3e-2


def _masked_lse(x, y, pot, logw, eps, keep):
    t = (2.0 / eps) * (x.double() @ y.double().T) + (pot.double() / eps + logw.double())[None]
    t = torch.where(keep, t, torch.full_like(t, -float("inf")))
    return -eps * torch.logsumexp(t, dim=1)


@pytest.mark.parametrize("mode", ["fp32", "tf32", "simt"])
@pytest.mark.parametrize("n,m,density,limit", [(300, 260, 0.7, 0), (3000, 2600, 0.3, 0), (3000, 2600, 0.3, 5),
                                               (5000, 900, 0.15, 0), (1300, 4000, 0.05, 148)])
def test_tile_lists_vs_dense_masked_fp64(monkeypatch, mode, n, m, density, limit):
    """Block-sparse alternating solve (kept 128 x 128 tiles as a CSR list, on the tensor cores in the fp32 and
    tf32 modes) against a dense masked fp64 loop: a few Gauss-Seidel iterations at two eps values. The masks
    always keep the diagonal band and hold at least one row block with a single kept tile; the forced CTA
    limits make one CTA cover many row blocks and many CTAs share one."""
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    monkeypatch.setenv("FLASH_SINKHORN_B200_PREC", mode)
    g = torch.Generator().manual_seed(n + m)
    d = 3
    x = (torch.rand(n, d, generator=g) * 2 - 1).cuda()
    y = (torch.rand(m, d, generator=g) * 2 - 1).cuda()
    a = torch.full((n,), 1.0 / n).cuda()
    b = torch.full((m,), 1.0 / m).cuda()
    nt, mt = (n + 127) // 128, (m + 127) // 128
    mask = torch.rand(nt, mt, generator=g) < density
    for i in range(nt):  # every row and column block keeps the tile on the (stretched) diagonal
        mask[i, min(mt - 1, i * mt // nt)] = True
    for j in range(mt):
        mask[min(nt - 1, j * nt // mt), j] = True
    mask[nt // 2, :] = False
    mask[nt // 2, min(mt - 1, (nt // 2) * mt // nt)] = True
    for j in range(mt):
        if not mask[:, j].any():
            mask[0, j] = True
    keep = mask.cuda().repeat_interleave(128, 0).repeat_interleave(128, 1)[:n, :m]
    stages, iters = [1.0, 0.3], 3
    la, lb = a.log(), b.log()
    xr, yr = (_tf32(x), _tf32(y)) if mode == "tf32" else (x, y)
    alpha, beta = (x.double() ** 2).sum(1), (y.double() ** 2).sum(1)
    fh, gh = -alpha, -beta
    for eps in stages:
        for _ in range(iters):
            fh = _masked_lse(xr, yr, gh, lb, eps, keep)
            gh = _masked_lse(yr, xr, fh, la, eps, keep.T)
    lib = _lib.load()
    previous = lib.fs_set_cta_limit(limit)
    try:
        f, gp = sinkhorn_flashstyle_alternating(x, y, a, b, eps_list=stages, iters_per_eps=iters, tile_mask=mask,
                                                allow_tf32=(mode == "tf32"))
        f2, _ = sinkhorn_flashstyle_alternating(x, y, a, b, eps_list=stages, iters_per_eps=iters, tile_mask=mask,
                                                allow_tf32=(mode == "tf32"))
    finally:
        lib.fs_set_cta_limit(previous)
    tol = 5e-3 if mode == "tf32" else 3e-4
    assert _r(f, fh + alpha) < tol and _r(gp, gh + beta) < tol
    assert torch.equal(f, f2)
    assert lib.fs_device_error() == 0


def test_row_block_without_kept_tiles_gets_the_empty_soft_min(monkeypatch):
    """A row block whose tile list is empty is visited by no work item; its rows must still be written (with
    the soft-min over nothing, +inf), identically on the tensor-core and the CUDA-core engine."""
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating
    g = torch.Generator().manual_seed(5)
    n, m = 700, 520
    x, y = torch.randn(n, 3, generator=g).cuda(), torch.randn(m, 3, generator=g).cuda()
    a, b = torch.full((n,), 1.0 / n).cuda(), torch.full((m,), 1.0 / m).cuda()
    mask = torch.ones((n + 127) // 128, (m + 127) // 128, dtype=torch.bool)
    mask[2, :] = False
    res = {}
    for mode in ("simt", "fp32"):
        monkeypatch.setenv("FLASH_SINKHORN_B200_PREC", mode)
        res[mode] = sinkhorn_flashstyle_alternating(x, y, a, b, eps=0.5, n_iters=1, tile_mask=mask, allow_tf32=False)
    for mode in res:
        f = res[mode][0]
        assert torch.isinf(f[256:384]).all() and (f[256:384] > 0).all()
        assert torch.isfinite(f[:256]).all() and torch.isfinite(f[384:]).all()
    assert _r(res["fp32"][0][:256], res["simt"][0][:256]) < 2e-4


def test_sharded_alternating_with_tile_lists_on_a_one_rank_group():
    """The multi-GPU block-sparse path (fs_symmetric_step_range_tiles, rows split by kept tiles, padded gather)
    on a one-rank NCCL group against the single-GPU solver; the two-rank loop with unequal ranges is covered
    on CPU (tests/test_sharded_gloo.py)."""
    import socket

    import torch.distributed as dist
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.distributed import alternating_solve_sharded
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_alternating, tile_mask_to_csr
    own_group = not dist.is_initialized()
    if own_group:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        g = torch.Generator().manual_seed(9)
        n, m = 1500, 1100
        x, y = (torch.rand(n, 3, generator=g)).cuda(), (torch.rand(m, 3, generator=g)).cuda()
        a, b = torch.full((n,), 1.0 / n).cuda(), torch.full((m,), 1.0 / m).cuda()
        nt, mt = (n + 127) // 128, (m + 127) // 128
        mask = torch.rand(nt, mt, generator=g) < 0.5
        mask[:, 0] = True
        mask[0, :] = True
        csr = tile_mask_to_csr(mask, x.device)
        counts = lambda t: [0] + torch.cumsum(t.sum(dim=1), dim=0).tolist()
        for prec, allow in ((_lib.PREC_FP32, False), (_lib.PREC_TF32, True)):
            f, gp, k = alternating_solve_sharded(
                x, y, a.log(), b.log(), [0.5, 0.1], 4, cost_scale=1.0, rho_x=None, rho_y=None, ott_convention=False,
                threshold=None, check_every=5, prec=prec, group=dist.group.WORLD, tile_csr=csr,
                tile_row_counts=(counts(mask), counts(mask.t())))
            f1, g1 = sinkhorn_flashstyle_alternating(x, y, a, b, eps_list=[0.5, 0.1], iters_per_eps=4, tile_mask=mask,
                                                     allow_tf32=allow)
            assert k == 8 and _r(f, f1) < 1e-5 and _r(gp, g1) < 1e-5
    finally:
        if own_group:
            dist.destroy_process_group()


@pytest.mark.parametrize("d,mode", [(64, "fp32"), (64, "tf32"), (24, "fp32"), (300, "tf32")])
def test_fused_multi_problem_step_with_packed_potentials(monkeypatch, d, mode):
    """fs_symmetric_step_multi on one GPU, playing both ranks of a two-rank layout in turn: three problems
    (cross term and two self-transport terms of a debiased loss, different sizes) advance one Jacobi step as one
    fused launch per "rank", reading and writing the packed [ranks, width] buffer. The result must equal the
    ordinary one-problem step (up to the order in which a row's partial sums merge)."""
    import ctypes

    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.distributed import PackedLayout, shard_range
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_symmetric_step
    monkeypatch.setenv("FLASH_SINKHORN_B200_PREC", mode)
    prec = _lib.precision_id(mode == "tf32")
    g = torch.Generator().manual_seed(d)
    n, m = 1500, 1100
    x = (torch.randn(n, d, generator=g) / d**0.5).cuda()
    y = (0.3 + torch.randn(m, d, generator=g) / d**0.5).cuda()
    a = torch.softmax(torch.randn(n, generator=g), 0).cuda()
    b = torch.softmax(torch.randn(m, generator=g), 0).cuda()
    eps, w, world = 0.2, 0.5, 2
    probs = [(x, y, a, b, False), (x, x, a, a, True), (y, y, b, b, True)]
    layout = PackedLayout([(p[0].shape[0], p[1].shape[0], p[4]) for p in probs], world)
    old, new = layout.new_buffer(x), layout.new_buffer(x)
    pots, wss = [], []
    for k, (px, py, pa, pb, selfp) in enumerate(probs):
        fh = -(px**2).sum(1) + 0.1 * torch.randn(px.shape[0], generator=g).cuda()
        gh = fh if selfp else -(py**2).sum(1) + 0.1 * torch.randn(py.shape[0], generator=g).cuda()
        layout.store(old, k, 0, fh)
        if not selfp:
            layout.store(old, k, 1, gh)
        pots.append((fh, gh))
        wss.append(_lib.workspace(_lib.OP_STEP, px.shape[0], py.shape[0], d, prec, x.device))
    fsz = 4
    keep = []
    for rank in range(world):
        arr = (_lib.StepItem * len(probs))()
        for k, (slot, (px, py, pa, pb, selfp)) in enumerate(zip(arr, probs)):
            (f_off, f_shard, _), (g_off, g_shard, _) = layout.slots[k]
            la, lb = pa.log().contiguous(), pb.log().contiguous()
            keep += [la, lb]
            f_lo, f_hi = shard_range(px.shape[0], world, rank)
            g_lo, g_hi = shard_range(py.shape[0], world, rank)
            if selfp:
                g_hi = g_lo
            slot.x, slot.y, slot.n, slot.m = px.data_ptr(), py.data_ptr(), px.shape[0], py.shape[0]
            slot.f_hat, slot.g_hat = old.data_ptr() + fsz * f_off, old.data_ptr() + fsz * g_off
            slot.f_out, slot.g_out = new.data_ptr() + fsz * f_off, new.data_ptr() + fsz * g_off
            slot.log_a, slot.log_b = la.data_ptr(), lb.data_ptr()
            slot.alpha_x, slot.beta_y = None, None
            slot.eps, slot.w, slot.damp_f, slot.damp_g, slot.cost_scale = eps, w, 1.0, 1.0, 1.0
            slot.f_begin, slot.f_end, slot.g_begin, slot.g_end = f_lo, f_hi, g_lo, g_hi
            slot.restage = 1 if rank == 0 else 0
            slot.ws, slot.ws_bytes = wss[k].data_ptr(), wss[k].numel()
            slot.f_shard, slot.g_shard, slot.pack_stride = f_shard, g_shard, layout.width
        _lib.call("fs_symmetric_step_multi", x.device, ctypes.cast(arr, ctypes.c_void_p), len(probs), d, prec,
                  _lib.stream_ptr(x.device))
    tol = 2e-3 if mode == "tf32" else 1e-5
    for k, (px, py, pa, pb, selfp) in enumerate(probs):
        fh, gh = pots[k]
        f1, g1 = flashsinkhorn_symmetric_step(px, py, fh, gh, pa.log(), pb.log(), eps, alpha=w, allow_tf32=(mode == "tf32"))
        assert _r(layout.full(new, k, 0), f1) < tol, (k, "f")
        if not selfp:
            assert _r(layout.full(new, k, 1), g1) < tol, (k, "g")
    assert _lib.load().fs_device_error() == 0


def test_fused_sharded_debiased_solves_on_a_one_rank_group(monkeypatch):
    """symmetric_solve_sharded_many (the multi-GPU path of a debiased loss) on a one-rank NCCL group: the fused
    lockstep schedule, the pass-by-pass schedule and the single-GPU solver agree."""
    import socket

    import torch.distributed as dist
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.distributed import symmetric_solve_sharded_many
    from flash_sinkhorn_b200.sinkhorn_solvers import sinkhorn_flashstyle_symmetric
    own_group = not dist.is_initialized()
    if own_group:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        g = torch.Generator().manual_seed(21)
        n, m, d = 900, 700, 32
        x, y = torch.randn(n, d, generator=g).cuda(), (0.5 + torch.randn(m, d, generator=g)).cuda()
        a, b = torch.full((n,), 1.0 / n).cuda(), torch.softmax(torch.randn(m, generator=g), 0).cuda()
        la, lb = a.log(), b.log()
        eps_list = [2.0, 1.0, 0.5, 0.5, 0.5]
        common = dict(cost_scale=0.5, rho_x=None, rho_y=2.0, last_extrapolation=True, threshold=None, check_every=5,
                      f_init=None, g_init=None, prec=_lib.PREC_FP32)
        probs = [dict(x=x, y=y, log_a=la, log_b=lb, eps_list=eps_list, **common),
                 dict(x=x, y=x, log_a=la, log_b=la, eps_list=eps_list[:3], **dict(common, rho_y=None)),
                 dict(x=y, y=y, log_a=lb, log_b=lb, eps_list=eps_list, **dict(common, rho_y=None))]
        fused = symmetric_solve_sharded_many(probs, group=dist.group.WORLD)
        monkeypatch.setenv("FLASH_SINKHORN_B200_FUSED_STEPS", "0")
        plain = symmetric_solve_sharded_many(probs, group=dist.group.WORLD)
        for fu, pl in zip(fused, plain):
            assert fu[4] == pl[4]
            for u, v in zip(fu[:4], pl[:4]):
                assert _r(u, v) < 1e-5
        f1, g1, fp1, gp1 = sinkhorn_flashstyle_symmetric(x, y, a, b, eps_list=eps_list, use_epsilon_scaling=False,
                                                         cost_scale=0.5, rho_y=2.0, allow_tf32=False, return_prelast=True)
        assert _r(fused[0][0], f1) < 1e-5 and _r(fused[0][1], g1) < 1e-5 and _r(fused[0][3], gp1) < 1e-5
    finally:
        if own_group:
            dist.destroy_process_group()


@pytest.mark.parametrize("d,tf32", [(64, False), (160, True), (100, True)])
def test_resident_and_streamed_kernels_agree_on_shapes_both_can_serve(d, tf32):
    """Shapes whose resident-operand plan only fits 64-column tiles run on the K-streamed kernels by default; the
    resident kernels stay selectable (`fs_set_prefer_streamed(0)`) and are what multi-pass launches use. Both
    contract the same staged operands in the same K order, so soft-mins and plan-times-vector agree to rounding."""
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_vec_flashstyle
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import flashsinkhorn_lse
    lib = _lib.load()
    g = torch.Generator().manual_seed(d)
    n, m = 1900, 2300
    x = (torch.randn(n, d, generator=g) / d**0.5).cuda()
    y = (torch.randn(m, d, generator=g) / d**0.5).cuda()
    bias = torch.randn(m, generator=g).cuda()
    la, lb = torch.full((n,), -math.log(n)).cuda(), torch.full((m,), -math.log(m)).cuda()
    gh = -(y**2).sum(1)
    v = torch.randn(m, generator=g).cuda()
    out = {}
    previous = lib.fs_set_prefer_streamed(1)
    try:
        for on in (1, 0):
            lib.fs_set_prefer_streamed(on)
            f = flashsinkhorn_lse(x, y, bias, 0.1, allow_tf32=tf32)
            fh = flashsinkhorn_lse(x, y, gh / 0.1 + lb, 0.1, allow_tf32=tf32)
            pv = apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, v, eps=0.1, axis=1, allow_tf32=tf32)
            out[on] = (f, pv)
    finally:
        lib.fs_set_prefer_streamed(previous)
    assert _r(out[1][0], out[0][0]) < 2e-6
    # plan-times-vector: the resident kernel rounds weights and vector to TF32 for its second GEMM in TF32 mode,
    # the K-streamed one multiplies them in fp32
    assert _r(out[1][1], out[0][1]) < (2e-3 if tf32 else 2e-5)
    assert lib.fs_device_error() == 0


@pytest.mark.parametrize("mode", ["fp32", "tf32"])
def test_batched_inputs_go_out_as_one_lockstep_solve(monkeypatch, mode):
    """(B, N, D) inputs: all solves of the batch (three per item with debiasing) run in one library call, several
    soft-min passes per launch. Loss and gradients equal the per-item loop up to the merge order of partial sums,
    with fewer launches; `potentials=True` returns the per-item potentials."""
    from flash_sinkhorn_b200 import SamplesLoss, _lib
    monkeypatch.setenv("FLASH_SINKHORN_B200_PREC", mode)
    tf32 = mode == "tf32"
    g = torch.Generator().manual_seed(17)
    B, n, m, d = 3, 600, 500, 24
    x = torch.randn(B, n, d, generator=g).cuda()
    y = (0.4 + torch.randn(B, m, d, generator=g) * torch.tensor([1.0, 1.5, 0.7]).view(B, 1, 1)).cuda()
    a = torch.softmax(torch.randn(B, n, generator=g), 1).cuda()
    b = torch.softmax(torch.randn(B, m, generator=g), 1).cuda()
    lib = _lib.load()
    for kw in (dict(blur=0.3, scaling=0.6, debias=True, half_cost=True),
               dict(blur=0.5, use_epsilon_scaling=False, eps=0.25, n_iters=12, reach=2.0, last_extrapolation=False)):
        loss = SamplesLoss("sinkhorn", allow_tf32=tf32, **kw)
        xs = x.clone().requires_grad_(True)
        c0 = lib.fs_launch_count()
        vals = loss(a, xs, b, y)
        batched_launches = lib.fs_launch_count() - c0
        (gx,) = torch.autograd.grad(vals.sum(), xs)
        assert vals.shape == (B,)
        c0 = lib.fs_launch_count()
        singles = []
        for i in range(B):
            xi = x[i].clone().requires_grad_(True)
            vi = loss(a[i], xi, b[i], y[i])
            (gi,) = torch.autograd.grad(vi, xi)
            singles.append((vi, gi))
        loop_launches = lib.fs_launch_count() - c0
        tol_l, tol_g = (1e-4, 3e-2) if tf32 else (1e-5, 2e-4)
        for i, (vi, gi) in enumerate(singles):
            assert abs(float(vals[i]) - float(vi)) <= tol_l * abs(float(vi)), (kw, i)
            assert _r(gx[i], gi) < tol_g, (kw, i)
        assert batched_launches < loop_launches
    pot = SamplesLoss("sinkhorn", blur=0.3, scaling=0.6, potentials=True, allow_tf32=tf32)
    f, gpot = pot(a, x, b, y)
    assert f.shape == (B, n) and gpot.shape == (B, m)
    f0, g0 = pot(a[1], x[1], b[1], y[1])
    assert _r(f[1], f0) < (2e-3 if tf32 else 1e-5) and _r(gpot[1], g0) < (2e-3 if tf32 else 1e-5)
    assert lib.fs_device_error() == 0
