"""The C++ accountant against independent computations that need nothing but NumPy / SciPy.

* Poisson-subsampled Gaussian, T-fold: a textbook privacy-loss-distribution composition written here from scratch
  (fine x-grid, losses binned once rounding up and once rounding down, FFT power) brackets the true epsilon from both
  sides; the accountant must land inside the bracket. Single steps are checked against adaptive quadrature of the
  hockey-stick integral. The integer-order Renyi bound of the sampled Gaussian mechanism must lie above the PLD value.
* Random allocation: brackets from an independent implementation of the same analysis (the values the reference pins in
  packages/opake-accounting/src/amplification/random_allocation.rs, test_golden_epsilons) and exact corner cases.
* Truncated Poisson: the two-component mixture of Ganesh (2025) evaluated by quadrature.
* b-min-sep Monte Carlo: corner cases with a closed form (one band = plain Poisson sampling; p = 1 = no sampling).
"""
import math

import numpy as np
import pytest
from scipy import integrate, special, stats

from opake_b200.accounting._native import native

N = native()


def _cfg(**kw):
    return N.DiscretizationConfig(**kw)


# ----------------------------------------------------------------------------------------------- independent PLD bracket
def _poisson_gaussian_bracket(sigma: float, q: float, T: int, delta: float, h: float = 4e-6):
    """(eps_low, eps_high): epsilon(delta) of the T-fold Poisson-subsampled Gaussian from a PLD built here, with losses
    rounded down / up to the grid ``h`` (remove and add directions, maximum of the two)."""
    span = 12.0 * sigma + 1.0
    x = np.linspace(-span, span + 1.0, 1_000_001)
    dx = x[1] - x[0]
    q0 = stats.norm.pdf(x, 0.0, sigma)
    p1 = stats.norm.pdf(x, 1.0, sigma)
    mix = (1 - q) * q0 + q * p1
    loss_rem = np.log(mix) - np.log(q0)          # sampled under the mixture
    w_rem = mix * dx
    loss_add = -loss_rem                          # sampled under q0
    w_add = q0 * dx

    def eps_of(loss, w, up):
        idx = np.ceil(loss / h - 1e-12) if up else np.floor(loss / h + 1e-12)
        idx = idx.astype(np.int64)
        lo = idx.min()
        pmf = np.bincount(idx - lo, weights=w)
        pmf /= pmf.sum()
        # drop 1e-13 of mass at either end (T times that is far below delta); the upper tail is re-added as if it were
        # an infinite loss when rounding up, the lower tail is moved onto the first kept point
        c = np.cumsum(pmf)
        first = int(np.searchsorted(c, 1e-13))
        last = int(np.searchsorted(c, 1.0 - 1e-13)) + 1
        tail_hi = float(pmf[last:].sum())
        head = float(pmf[:first].sum())
        pmf = pmf[first:last].copy()
        pmf[0] += head
        lo += first
        n = len(pmf)
        size = 1 << int(np.ceil(np.log2(n * T)))
        f = np.fft.rfft(pmf, size)
        comp = np.fft.irfft(f ** T, size)[: (n - 1) * T + 1]
        comp = np.maximum(comp, 0.0)
        losses = (lo * T + np.arange(len(comp))) * h
        # delta(eps) = sum_{l > eps} p (1 - e^{eps - l}); find eps by bisection
        order = np.argsort(losses)
        losses, comp = losses[order], comp[order]
        csum = np.cumsum(comp[::-1])[::-1]
        cexp = np.cumsum((comp * np.exp(-losses))[::-1])[::-1]

        extra = T * tail_hi if up else 0.0

        def dlt(e):
            k = np.searchsorted(losses, e, side="right")
            if k >= len(losses):
                return extra
            return extra + csum[k] - math.exp(e) * cexp[k]

        a, b = 0.0, 50.0
        for _ in range(80):
            m = 0.5 * (a + b)
            if dlt(m) > delta:
                a = m
            else:
                b = m
        return 0.5 * (a + b)

    low = max(eps_of(loss_rem, w_rem, False), eps_of(loss_add, w_add, False))
    high = max(eps_of(loss_rem, w_rem, True), eps_of(loss_add, w_add, True))
    return low, high


@pytest.mark.parametrize("sigma,q,T,delta", [(0.8, 0.05, 10, 1e-6), (1.1, 256 / 60000, 50, 1e-5), (2.0, 0.1, 20, 1e-6)])
def test_poisson_gaussian_epsilon_inside_independent_bracket(sigma, q, T, delta):
    cfg = _cfg(discretization=2e-5)
    got = N.poisson_pld(N.gaussian_pld(sigma, cfg), q).self_compose(T).epsilon_at(delta)
    low, high = _poisson_gaussian_bracket(sigma, q, T, delta)
    assert high - low < 2.5e-4, (low, high)
    assert low - 1e-4 <= got <= high + 4e-4 * max(1, T ** 0.5), (got, low, high)
    # the accountant rounds pessimistically: never below the optimistic end of the bracket
    assert got >= low - 1e-6


@pytest.mark.parametrize("sigma,q", [(0.7, 0.02), (1.3, 0.2), (3.0, 0.5)])
def test_single_step_delta_matches_quadrature(sigma, q):
    pld = N.poisson_pld(N.gaussian_pld(sigma, _cfg(discretization=1e-5)), q)
    for eps in (0.05, 0.3, 1.0):
        def f_rem(x):
            m = (1 - q) * stats.norm.pdf(x, 0, sigma) + q * stats.norm.pdf(x, 1, sigma)
            return max(0.0, m - math.exp(eps) * stats.norm.pdf(x, 0, sigma))

        def f_add(x):
            m = (1 - q) * stats.norm.pdf(x, 0, sigma) + q * stats.norm.pdf(x, 1, sigma)
            return max(0.0, stats.norm.pdf(x, 0, sigma) - math.exp(eps) * m)

        want = max(integrate.quad(f_rem, -15 * sigma, 15 * sigma + 1, limit=400, points=[0, 1])[0],
                   integrate.quad(f_add, -15 * sigma, 15 * sigma + 1, limit=400, points=[0, 1])[0])
        got = pld.delta_at(eps)
        assert got >= want - 2e-8
        assert got - want < 3e-5 * max(want, 1e-3) + 2e-7, (eps, got, want)


def _rdp_epsilon(sigma, q, T, delta):
    """Integer-order Renyi bound of the sampled Gaussian mechanism (Mironov, Talwar, Zhang 2019), converted with the
    standard eps = rdp + log(1/delta) / (alpha - 1)."""
    best = math.inf
    for a in range(2, 256):
        terms = [math.log(special.comb(a, k)) + (a - k) * math.log1p(-q) + k * math.log(q) + (k * k - k) / (2 * sigma ** 2)
                 for k in range(a + 1)]
        log_a = special.logsumexp(terms)
        best = min(best, T * log_a / (a - 1) + math.log(1 / delta) / (a - 1))
    return best


@pytest.mark.parametrize("sigma,q,T", [(1.0, 0.01, 1000), (0.9, 256 / 50000, 4000), (1.5, 0.05, 200)])
def test_pld_epsilon_below_renyi_bound(sigma, q, T):
    delta = 1e-5
    got = N.poisson_pld(N.gaussian_pld(sigma, _cfg()), q).self_compose(T).epsilon_at(delta)
    rdp = _rdp_epsilon(sigma, q, T, delta)
    assert 0.3 * rdp < got <= rdp, (got, rdp)


# ----------------------------------------------------------------------------------------------- random allocation
@pytest.mark.parametrize("sigma,t,lo,hi", [(1.0, 8, 3.711, 3.727), (1.0, 64, 1.792, 1.807)])
def test_random_allocation_inside_independent_brackets(sigma, t, lo, hi):
    got = N.random_allocation_gaussian_pld(sigma, t, 1, _cfg()).epsilon_at(1e-8)
    assert lo <= got <= hi, got


def test_random_allocation_corner_cases_and_monotonicity():
    cfg = _cfg(max_conv_grid=8192)
    base = N.gaussian_pld(1.0, cfg).epsilon_at(1e-8)
    assert N.random_allocation_gaussian_pld(1.0, 1, 1, cfg).epsilon_at(1e-8) == pytest.approx(base, rel=1e-9)
    e = [N.random_allocation_gaussian_pld(1.0, t, 1, cfg).epsilon_at(1e-8) for t in (2, 4, 16)]
    assert base > e[0] > e[1] > e[2]                                       # more steps to hide among
    assert N.random_allocation_gaussian_pld(2.0, 16, 1, cfg).epsilon_at(1e-8) < e[2]      # more noise
    e4 = N.random_allocation_gaussian_pld(1.0, 16, 4, cfg).epsilon_at(1e-8)
    assert e4 > e[2]                                                       # more participations
    # k = t: the record is used in every step, i.e. the plain t-fold Gaussian composition
    all_steps = N.random_allocation_gaussian_pld(1.0, 4, 4, cfg).epsilon_at(1e-8)
    assert all_steps == pytest.approx(N.gaussian_pld(0.5, cfg).epsilon_at(1e-8), rel=2e-3)
    # deterministic: no Monte-Carlo failure probability attached
    assert N.random_allocation_gaussian_pld(1.0, 8, 1, cfg).mc_failure_probability == 0.0


def test_random_allocation_matches_direct_sampling():
    """Empirical delta(eps) of the 1-of-t allocation from one million direct draws of the likelihood ratio."""
    sigma, t, eps = 1.2, 12, 0.8
    rng = np.random.default_rng(0)
    n = 1_000_000
    mu, s = 0.5 / sigma ** 2, 1.0 / sigma
    terms = rng.normal(-mu, s, size=(n, t))
    terms[:, 0] = rng.normal(mu, s, size=n)
    loss = special.logsumexp(terms, axis=1) - math.log(t)
    emp = np.mean(np.maximum(0.0, 1.0 - np.exp(eps - loss)))
    got = N.random_allocation_gaussian_pld(sigma, t, 1, _cfg(max_conv_grid=8192)).delta_at(eps)
    assert got >= emp - 4 * math.sqrt(emp / n)
    assert got <= emp * 1.05 + 1e-4, (got, emp)


# ----------------------------------------------------------------------------------------------- truncated Poisson
def test_truncated_poisson_is_the_two_component_mixture():
    sigma, q, cap, n = 0.9, 0.02, 230, 10_000
    pld = N.truncated_poisson_gaussian_pld(sigma, q, cap, n, _cfg(discretization=1e-5))
    p_trunc = stats.binom.sf(cap - 1, n - 1, q)
    q_cond = stats.binom.sf(cap, n, q) * cap / n / p_trunc
    assert 0 < p_trunc < 0.05 and 0 < q_cond < 1
    plain = N.poisson_pld(N.gaussian_pld(sigma, _cfg(discretization=1e-5)), q)
    for eps in (0.1, 0.5, 1.5):
        d = 2.0 / sigma

        def f(x):
            a = (1 - q_cond) * stats.norm.pdf(x) + q_cond * stats.norm.pdf(x - d)
            b = (1 - q_cond) * stats.norm.pdf(x) + q_cond * stats.norm.pdf(x + d)
            return max(0.0, a - math.exp(eps) * b)

        comp2 = integrate.quad(f, -40, 40, limit=400, points=[-d, 0, d])[0]
        want = (1 - p_trunc) * plain.delta_at(eps) + p_trunc * comp2
        got = pld.delta_at(eps)
        assert got == pytest.approx(want, rel=2e-3, abs=1e-8), (eps, got, want)


def test_truncated_poisson_limits():
    cfg = _cfg()
    plain = N.poisson_pld(N.gaussian_pld(1.0, cfg), 0.01).self_compose(50).epsilon_at(1e-5)
    loose = N.truncated_poisson_gaussian_pld(1.0, 0.01, 5000, 10_000, cfg).self_compose(50).epsilon_at(1e-5)
    assert loose == pytest.approx(plain, rel=1e-6)                 # a cap that never binds changes nothing
    e = [N.truncated_poisson_gaussian_pld(1.0, 0.01, cap, 10_000, cfg).self_compose(50).epsilon_at(1e-5) for cap in (140, 120, 100)]
    assert plain <= e[0] <= e[1] <= e[2]                           # a tighter cap costs privacy
    with pytest.raises(ValueError):
        N.truncated_poisson_gaussian_pld(1.0, 0.01, 0, 100, cfg)


# ----------------------------------------------------------------------------------------------- b-min-sep Monte Carlo
def test_b_min_sep_monte_carlo_corner_cases():
    cfg = _cfg(mc_resolution=2e-4)
    delta = 1e-3
    # one band, p = 1: every step takes part: n-fold Gaussian composition
    n, sigma = 16, 4.0
    got = N.bandmf_b_min_sep_warm_mc_pld([1.0], n, 1.0, sigma, cfg).epsilon_at(delta)
    want = N.gaussian_pld(sigma / math.sqrt(n), cfg).epsilon_at(delta)
    assert got == pytest.approx(want, rel=0.06)
    # one band, p < 1: independent Poisson sampling in every step
    got = N.bandmf_b_min_sep_warm_mc_pld([1.0], 32, 0.1, 1.0, cfg).epsilon_at(delta)
    want = N.poisson_pld(N.gaussian_pld(1.0, cfg), 0.1).self_compose(32).epsilon_at(delta)
    assert got == pytest.approx(want, rel=0.08)
    # several bands: sampling amplifies, so the estimate lies below the un-amplified worst-case participation bound
    coef = [1.0, 0.5, 0.375, 0.3125]
    amplified = N.bandmf_b_min_sep_warm_mc_pld(coef, 64, 0.05, 2.0, cfg)
    sens2 = N.toeplitz_minsep_sensitivity_squared(coef, 64, 4, None)
    bound = N.gaussian_pld(2.0 / math.sqrt(sens2), cfg).epsilon_at(delta)
    assert 0 < amplified.epsilon_at(delta) < bound
    assert amplified.mc_failure_probability > 0
    # a registered corpus gives the same estimate for the same seed and serves several noise levels
    h = N.register_b_min_sep_transcript_corpus(coef, 64, 0.05, cfg.resolved_num_mc_samples, cfg.seed)
    again = N.bandmf_b_min_sep_pld_from_transcript_handle(h, coef, 0.05, 2.0, cfg).epsilon_at(delta)
    quieter = N.bandmf_b_min_sep_pld_from_transcript_handle(h, coef, 0.05, 4.0, cfg).epsilon_at(delta)
    N.drop_b_min_sep_transcript_corpus(h)
    assert again == pytest.approx(amplified.epsilon_at(delta), rel=1e-12) and quieter < again


def test_learning_rate_weighted_gram_functions_raise_like_the_reference():
    with pytest.raises(ValueError):
        N.bisr_gram_matrix_lr([1.0, 0.5], 0.0, 8, 2, None, True, [1.0] * 8)
    with pytest.raises(ValueError):
        N.lambda_cgd_gram_matrix_lr(0.5, 0.0, 8, 2, None, True, [1.0] * 8)


def test_cyclic_banded_cholesky_matches_the_dense_factor():
    """The balls-in-bins sampler factors the Gram matrix over bins, which is banded modulo the number of bins (corner
    blocks included). The structured factor keeps the band plus dense trailing rows; it must reproduce the dense
    Cholesky factor, detect the CYCLIC (not the linear) bandwidth, and fall back to dense for unstructured input."""
    import numpy as np

    from opake_b200.accounting._native import native

    N = native()

    def cyclic_gram(b, width):
        # G = C^T C for a circulant C with `width` sub-diagonals (wrapping around): cyclic bandwidth `width`, and
        # positive definite because C is strictly diagonally dominant
        col = np.zeros(b)
        col[0] = 3.0
        col[1 : width + 1] = 0.9 ** np.arange(1, width + 1)
        C = np.stack([np.roll(col, j) for j in range(b)], axis=1)
        return C.T @ C

    for b, width in ((24, 3), (40, 5), (17, 2)):
        G = cyclic_gram(b, width)
        assert np.linalg.eigvalsh(G).min() > 0
        p, L = N.cyclic_banded_cholesky(G.reshape(-1).tolist(), b)
        L = np.asarray(L).reshape(b, b)
        assert p == width                                                   # the corner entries count with distance b - |i-j|
        assert np.allclose(L, np.linalg.cholesky(G), atol=1e-10)
        assert np.allclose(L @ L.T, G, atol=1e-10)
        # structure: band rows hold nothing left of the band, the last `width` rows are dense
        for i in range(b - width):
            assert np.all(L[i, : max(0, i - width)] == 0.0)
        assert np.abs(L[b - 1, :width]).max() > 0                           # the corner block fills in
    rng = np.random.default_rng(0)
    A = rng.normal(size=(9, 9))
    G = A @ A.T + 9 * np.eye(9)
    p, L = N.cyclic_banded_cholesky(G.reshape(-1).tolist(), 9)
    assert p == 4 and np.allclose(np.asarray(L).reshape(9, 9), np.linalg.cholesky(G), atol=1e-10)
    with pytest.raises(ValueError):
        N.cyclic_banded_cholesky([1.0, 0.0, 0.0], 2)
