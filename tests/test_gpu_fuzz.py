"""Seeded random shapes (1 <= n, m <= 4000, d from 1 to 257, both precisions, both cost scalings) through the
single-pass entry points, each against dense float64 torch on the same device. Errors are measured against the
size of the summed terms, so that outputs which cancel to almost nothing do not inflate them."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DIMS = [1, 2, 3, 5, 8, 16, 31, 64, 100, 128, 200, 257]


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _err(got, want, size):
    return float(((got.double() - want).abs() / size.clamp_min(1e-30)).max())


@pytest.mark.parametrize("seed", [11, 12])
def test_random_shapes_vs_dense(seed):
    from flash_sinkhorn_b200 import _lib
    from flash_sinkhorn_b200.kernels.apply_flash import apply_plan_mat_flashstyle, apply_plan_vec_flashstyle
    from flash_sinkhorn_b200.kernels.c_transform_sqeuclid import c_transform_kernel
    from flash_sinkhorn_b200.kernels.grad_sqeuclid import sinkhorn_geomloss_online_grad_sqeuclid
    from flash_sinkhorn_b200.kernels.sinkhorn_flashstyle_sqeuclid import (
        flashsinkhorn_lse, flashsinkhorn_symmetric_step)
    g = torch.Generator().manual_seed(seed)

    def log_uniform(lo, hi):
        u = torch.rand((), generator=g).item()
        return int(math.exp(u * (math.log(hi) - math.log(lo)) + math.log(lo)))

    worst = {}
    for case in range(120):
        n, m = log_uniform(1, 4000), log_uniform(1, 4000)
        d = DIMS[int(torch.randint(len(DIMS), (), generator=g))]
        eps = float(0.1 + 2 * torch.rand((), generator=g))
        cs = [0.5, 1.0][int(torch.randint(2, (), generator=g))]
        tf32 = bool(torch.randint(2, (), generator=g))
        tol = 3e-2 if tf32 else 2e-4
        sc = 1.0 / math.sqrt(d)
        x = (sc * torch.randn(n, d, generator=g)).cuda()
        y = (0.1 + sc * torch.randn(m, d, generator=g)).cuda()
        a = torch.softmax(torch.randn(n, generator=g), 0).cuda()
        b = torch.softmax(torch.randn(m, generator=g), 0).cuda()
        fh = -cs * (x * x).sum(1) + 0.1 * torch.randn(n, generator=g).cuda()
        gh = -cs * (y * y).sum(1) + 0.1 * torch.randn(m, generator=g).cuda()
        vm, vn = torch.randn(m, generator=g).cuda(), torch.randn(n, generator=g).cuda()
        Mm, Mn = torch.randn(m, d, generator=g).cuda(), torch.randn(n, d, generator=g).cuda()
        psi = torch.randn(m, generator=g).cuda()
        la, lb = a.log(), b.log()
        X, Y = x.double(), y.double()
        S = (2 * cs / eps) * (X @ Y.T)
        kw = dict(cost_scale=cs, allow_tf32=tf32)
        errs = {}

        bias = gh / eps + lb
        want = -eps * torch.logsumexp(S + bias.double()[None, :], 1)
        errs["lse"] = _err(flashsinkhorn_lse(x, y, bias, eps, **kw), want, 1 + want.abs())
        sf, sg = flashsinkhorn_symmetric_step(x, y, fh, gh, la, lb, eps, alpha=0.5, damping_f=0.9, **kw)
        cf = -eps * 0.9 * torch.logsumexp(S + (gh.double() / eps + lb.double())[None, :], 1)
        cg = -eps * torch.logsumexp(S.T + (fh.double() / eps + la.double())[None, :], 1)
        errs["step_f"] = _err(sf, 0.5 * fh.double() + 0.5 * cf, 1 + cf.abs())
        errs["step_g"] = _err(sg, 0.5 * gh.double() + 0.5 * cg, 1 + cg.abs())

        P = torch.exp(S + (fh.double() / eps + la.double())[:, None] + (gh.double() / eps + lb.double())[None, :])
        akw = dict(eps=eps, **kw)
        errs["vec1"] = _err(apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, vm, axis=1, **akw), P @ vm.double(),
                            P @ vm.double().abs())
        errs["vec0"] = _err(apply_plan_vec_flashstyle(x, y, fh, gh, la, lb, vn, axis=0, **akw), P.T @ vn.double(),
                            P.T @ vn.double().abs())
        errs["mat1"] = _err(apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, Mm, axis=1, **akw), P @ Mm.double(),
                            (P @ Mm.double().abs()).amax(1, keepdim=True))
        errs["mat0"] = _err(apply_plan_mat_flashstyle(x, y, fh, gh, la, lb, Mn, axis=0, **akw), P.T @ Mn.double(),
                            (P.T @ Mn.double().abs()).amax(1, keepdim=True))

        f, gg = fh + cs * (x * x).sum(1), gh + cs * (y * y).sum(1)
        gx, gy = sinkhorn_geomloss_online_grad_sqeuclid(x, y, a, b, f, gg, eps=eps, **kw)
        C = cs * ((X * X).sum(1)[:, None] + (Y * Y).sum(1)[None, :] - 2 * X @ Y.T)
        Wx = torch.softmax((gg.double()[None, :] - C) / eps + lb.double()[None, :], 1)
        Wy = torch.softmax((f.double()[:, None] - C) / eps + la.double()[:, None], 0)
        size_x = 2 * cs * a.double()[:, None] * (X.abs() + Wx @ Y.abs()).amax(1, keepdim=True)
        size_y = 2 * cs * b.double()[:, None] * (Y.abs() + Wy.T @ X.abs()).amax(1, keepdim=True)
        errs["grad_x"] = _err(gx, 2 * cs * a.double()[:, None] * (X - Wx @ Y), size_x)
        errs["grad_y"] = _err(gy, 2 * cs * b.double()[:, None] * (Y - Wy.T @ X), size_y)

        cbias = cs * (y * y).sum(1) - psi
        cv, ci = c_transform_kernel(x, y, cbias, **kw)
        full = -2 * cs * (X @ Y.T) + cbias.double()[None, :]
        wv = full.min(1).values
        picked = full.gather(1, ci.long()[:, None])[:, 0]
        errs["ct_value"] = _err(cv, wv, 1 + wv.abs())
        errs["ct_picked"] = _err(picked, wv, 1 + wv.abs())  # the chosen column attains the minimum

        assert _lib.load().fs_device_error() == 0
        for k, v in errs.items():
            assert v == v and v < tol, f"case {case} n={n} m={m} d={d} eps={eps:.3f} cs={cs} tf32={tf32}: {k}={v:.3e}"
            worst[(k, tf32)] = max(worst.get((k, tf32), 0.0), v)
    print({f"{k}/{'tf32' if t else 'fp32'}": f"{v:.1e}" for (k, t), v in sorted(worst.items())})
