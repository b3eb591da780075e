"""Properties the CPU oracle must have independently of any fixture (known-answer style checks the reference's
own tests use: marginals of a converged plan, self-divergence, half-cost ratio, cost-scale equivalence), plus
finite-difference checks of its gradient and Hessian-vector product. CPU only, float64, small sizes."""
import numpy as np
import pytest

from oracle import dense_sinkhorn as O


def _clouds(seed, n=40, m=33, d=3):
    rng = np.random.default_rng(seed)
    x, y = rng.normal(size=(n, d)), 0.3 + rng.normal(size=(m, d))
    a, b = rng.random(n) + 0.2, rng.random(m) + 0.2
    return x, y, a / a.sum(), b / b.sum()


def test_converged_balanced_plan_has_the_marginals():
    x, y, a, b = _clouds(0)
    eps = 0.5
    s = O.solve_symmetric(x, y, a, b, [eps] * 400)
    fo, go = s["f"] + eps * np.log(a), s["g"] + eps * np.log(b)
    P = O.plan_ott(x, y, fo, go, eps)
    assert np.abs(P.sum(1) - a).max() < 1e-9 and np.abs(P.sum(0) - b).max() < 1e-9
    # the dual value equals the primal transport cost plus eps * KL(P | a x b)
    C = O.sqnorm(x)[:, None] + O.sqnorm(y)[None, :] - 2 * x @ y.T
    primal = (P * C).sum() + eps * (P * (np.log(P) - np.log(a)[:, None] - np.log(b)[None, :])).sum()
    assert abs(O.ot_cost(a, b, s["f"], s["g"], eps) - primal) < 1e-8
    # alternating iterations reach the same potentials up to the additive constant
    alt = O.solve_alternating(x, y, a, b, [eps], 400)
    shift = np.mean(alt["f"] - s["f"])
    assert np.abs(alt["f"] - s["f"] - shift).max() < 1e-8 and np.abs(alt["g"] - s["g"] + shift).max() < 1e-8


def test_self_divergence_is_zero_and_self_potentials_coincide():
    x, _, a, _ = _clouds(1)
    out = O.samples_loss(x, x, a, a, [0.3] * 150, debias=True)
    assert abs(out["loss"]) < 1e-12
    s = O.solve_symmetric(x, x, a, a, [0.3] * 20)
    assert np.array_equal(s["f"], s["g"])  # the shortcut the engine uses for OT(x,x)


def test_half_cost_ratio_and_cost_scale_equivalence():
    x, y, a, b = _clouds(2)
    # doubling the cost and the temperature doubles every potential, hence the value: exact at every iterate
    full = O.samples_loss(x, y, a, b, [0.1] * 50, cost_scale=1.0)["loss"]
    half = O.samples_loss(x, y, a, b, [0.05] * 50, cost_scale=0.5)["loss"]
    assert abs(full - 2.0 * half) < 1e-12 * abs(full)
    # the reference's own check (testing/test_half_cost.py:11-33): 100 + 100 points in 32 dimensions,
    # blur 0.1 with the default annealing -> the cost dominates the entropy term and the ratio is close to 2
    rng = np.random.default_rng(42)
    xr, yr = rng.normal(size=(100, 32)), rng.normal(size=(100, 32))
    w = np.full(100, 0.01)
    sched = O.epsilon_schedule(O.max_diameter(xr, yr), 0.1, 0.5)
    full = O.samples_loss(xr, yr, w, w, sched, cost_scale=1.0)["loss"]
    half = O.samples_loss(xr, yr, w, w, sched, cost_scale=0.5)["loss"]
    assert 1.95 < full / half < 2.05
    # cost_scale cs on (x, y) is the unscaled problem on sqrt(cs) * (x, y), exactly
    scaled = O.solve_symmetric(np.sqrt(0.5) * x, np.sqrt(0.5) * y, a, b, [0.2] * 30, cost_scale=1.0)
    direct = O.solve_symmetric(x, y, a, b, [0.2] * 30, cost_scale=0.5)
    assert np.abs(scaled["f"] - direct["f"]).max() < 1e-12


def test_translation_invariance_and_symmetry():
    x, y, a, b = _clouds(3)
    base = O.samples_loss(x, y, a, b, [0.4] * 60, debias=True)["loss"]
    moved = O.samples_loss(x + 1.7, y + 1.7, a, b, [0.4] * 60, debias=True)["loss"]
    swapped = O.samples_loss(y, x, b, a, [0.4] * 60, debias=True)["loss"]
    assert abs(base - moved) < 1e-10 and abs(base - swapped) < 1e-10


@pytest.mark.parametrize("rho", [None, 1.5])
def test_gradient_matches_finite_differences_of_the_converged_cost(rho):
    x, y, a, b = _clouds(4, n=12, m=10, d=2)
    eps_list = [0.6] * 600

    def cost(xx):
        s = O.solve_symmetric(xx, y, a, b, eps_list, rho_x=rho, rho_y=rho)
        return O.ot_cost(a, b, s["f"], s["g"], 0.6, rho, rho)

    s = O.solve_symmetric(x, y, a, b, eps_list, rho_x=rho, rho_y=rho)
    gx, _ = O.grad_xy(x, y, a, b, s["f_pre"], s["g_pre"], 0.6)
    if rho is not None:
        # relaxed marginals: the envelope gradient carries the transported mass, a_i * exp(-f_i / rho)
        gx = gx * np.exp(-s["f_pre"] / rho)[:, None]
    h = 1e-5
    for (i, k) in ((0, 0), (5, 1), (11, 0)):
        e = np.zeros_like(x)
        e[i, k] = h
        fd = (cost(x + e) - cost(x - e)) / (2 * h)
        assert abs(fd - gx[i, k]) < 2e-6 * max(1.0, abs(fd)), (i, k, fd, gx[i, k])


def test_hvp_matches_finite_differences_of_the_gradient():
    x, y, a, b = _clouds(5, n=10, m=9, d=2)
    eps = 0.7
    eps_list = [eps] * 800

    def grad(xx):
        s = O.solve_symmetric(xx, y, a, b, eps_list)
        return O.grad_xy(xx, y, a, b, s["f"], s["g"], eps)[0]

    s = O.solve_symmetric(x, y, a, b, eps_list)
    fo, go = s["f"] + eps * np.log(a), s["g"] + eps * np.log(b)
    rng = np.random.default_rng(6)
    A = rng.normal(size=x.shape)
    hv = O.hvp_x(x, y, fo, go, A, eps, tau2=0.0, max_cg_iter=500, cg_rtol=1e-13, cg_atol=1e-13)["hvp"]
    h = 1e-5
    fd = (grad(x + h * A) - grad(x - h * A)) / (2 * h)
    assert np.abs(hv - fd).max() < 1e-5 * max(1.0, np.abs(fd).max())
