"""Privacy lower bounds from one training run (packages/opake-auditing/src/opake/api/auditing/one_run/
_estimate.py:47-354, _eps_delta.py:42-124, _gdp.py:55-438, _roc.py:17-121).

The attacker guesses membership of ``m`` coin-flipped canaries from their scores. Two estimators turn the number of
wrong guesses into a statement about the mechanism:

* ``EpsDeltaMethod`` (Steinke, Nasr, Jagielski 2023): under (eps, delta)-DP the number of mistakes stochastically
  dominates ``Binomial(m - round(m * delta), 1 / (1 + e^eps))``; the largest eps whose p-value stays below the
  significance level is a lower bound.
* ``GdpMethod``: the same test under mu-Gaussian-DP. For a mu-GDP pair the attacker who ranks canaries by absolute
  privacy loss errs on the k-th most confident guess with a probability ``v_k`` that is an order-statistic integral
  over the mixture density; the mistake count is Poisson-binomial and its lower tail is bounded by Chernoff.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import scipy.special
import scipy.stats

from ..base.exceptions import ConfigurationError, OperationError
from .coin_flip import CanaryScores, CoinFlip

__all__ = ["OneRunEstimate", "EpsDeltaMethod", "GdpMethod", "one_run", "get_tn_fn_counts", "pareto_frontier",
           "tpr_at_given_fpr"]


# ------------------------------------------------------------------------------------------------ ROC helpers
def pareto_frontier(points: np.ndarray) -> np.ndarray:
    """Indices of the upper-left convex hull of points sorted by x (drops points on or under a chord)."""
    if points.ndim != 2 or points.shape[0] < 2 or points.shape[1] != 2:
        raise ConfigurationError(f"Expected at least two 2D points, got shape {points.shape}")
    if not np.all(points[:-1, 0] <= points[1:, 0]):
        raise ConfigurationError("Expected points to be sorted by x-coordinate")
    hull: list[int] = []
    for i in range(points.shape[0]):
        while len(hull) >= 2:
            a, b = points[hull[-2]], points[hull[-1]]
            cross = (b[1] - a[1]) * (points[i][0] - b[0]) - (points[i][1] - b[1]) * (b[0] - a[0])
            if cross <= 0:
                hull.pop()
            else:
                break
        hull.append(i)
    return np.asarray(hull)


def get_tn_fn_counts(in_scores, out_scores, *, hull: bool = False):
    """For every threshold (each distinct score, then +inf): members scored below it (false negatives) and
    non-members scored below it (true negatives)."""
    a, b = np.asarray(in_scores), np.asarray(out_scores)
    if a.size == 0 and b.size == 0:
        raise ConfigurationError("At least one of the canary score arrays must be non-empty")
    thr = np.concatenate((np.union1d(a, b), [np.inf]))
    fn = np.searchsorted(np.sort(a), thr, side="left")
    tn = np.searchsorted(np.sort(b), thr, side="left")
    fn[-1], tn[-1] = a.size, b.size
    if hull:
        keep = pareto_frontier(np.stack([fn, tn], axis=1))
        return thr[keep], tn[keep], fn[keep]
    return thr, tn, fn


def tpr_at_given_fpr(fpr, tp_counts, fp_counts):
    """Linear interpolation of the empirical ROC at the requested false-positive rate(s)."""
    f = np.asarray(fpr)
    if not np.all((f >= 0) & (f <= 1)):
        raise ConfigurationError(f"fpr must be in [0, 1], got {fpr}")
    target = fp_counts[-1] * f
    hi = np.minimum(np.searchsorted(fp_counts, target, side="right"), np.size(fp_counts) - 1)
    left, right = fp_counts[hi - 1], fp_counts[hi]
    width = right - left
    frac = np.where(width > 0, (target - left) / np.where(width > 0, width, 1), 1.0)
    out = (tp_counts[hi - 1] + frac * (tp_counts[hi] - tp_counts[hi - 1])) / tp_counts[-1]
    return float(out) if np.isscalar(fpr) else out


def _auc(tn, fn) -> float:
    tnr, fnr = tn / tn[-1], fn / fn[-1]
    return float(0.5 * np.dot(tnr[:-1] + tnr[1:], fnr[1:] - fnr[:-1]))


# ------------------------------------------------------------------------------------------------ validation
def _check_significance(s: float) -> None:
    if not 0 < s < 0.5:
        raise ConfigurationError(f"significance must be in (0, 0.5), got {s}")


def _check_delta(d: float) -> None:
    if not 0 <= d <= 1:
        raise ConfigurationError(f"delta must be in [0, 1], got {d}")


def _search_ceiling(m: int, delta: float, significance: float) -> float:
    """Upper end of the bisection bracket: the eps at which even zero mistakes stop being significant, plus 10 %."""
    n_eff = max(m - round(m * delta), 1)
    return max(-math.log(significance ** (-1.0 / n_eff) - 1.0) * 1.1, 1.0)


# ------------------------------------------------------------------------------------------------ (eps, delta)
def _binom_p_value(m: int, mistakes: int, eps: float, delta: float) -> float:
    q = math.exp(-eps) if eps > 0 else 1.0
    n_eff = max(m - round(m * delta), 0)
    return 1.0 if n_eff == 0 else float(scipy.stats.binom.cdf(mistakes, n_eff, q / (1.0 + q)))


@dataclasses.dataclass(frozen=True)
class EpsDeltaMethod:
    _estimate: "OneRunEstimate"

    def epsilon_at(self, *, delta: float = 0.0, significance: float = 0.05, threshold: float | None = None) -> float:
        _check_significance(significance)
        _check_delta(delta)
        m, wrong = self._estimate._best_r_u(threshold)
        lo, hi = 0.0, _search_ceiling(m, delta, significance)
        while hi - lo > 1e-4:
            mid = 0.5 * (lo + hi)
            if _binom_p_value(m, wrong, mid, delta) < significance:
                lo = mid
            else:
                hi = mid
        return lo

    def delta_at(self, *, epsilon: float, significance: float = 0.05, threshold: float | None = None) -> float:
        _check_significance(significance)
        if epsilon < 0:
            raise ConfigurationError(f"epsilon must be >= 0, got {epsilon}")
        m, wrong = self._estimate._best_r_u(threshold)
        if _binom_p_value(m, wrong, epsilon, 0.0) >= significance:
            return 0.0
        lo, hi = 0.0, 1.0
        while hi - lo > 1e-6:
            mid = 0.5 * (lo + hi)
            if _binom_p_value(m, wrong, epsilon, mid) < significance:
                lo = mid
            else:
                hi = mid
        return lo


# ------------------------------------------------------------------------------------------------ mu-GDP
def _gdp_delta(mu: float, eps: float) -> float:
    t = eps + scipy.stats.norm.logcdf(-mu / 2.0 - eps / mu)
    return float(scipy.stats.norm.cdf(mu / 2.0 - eps / mu) - (math.exp(t) if t < 700 else math.inf))


def _gdp_to_eps(mu: float, delta: float) -> float:
    if mu < 0:
        raise ConfigurationError(f"mu must be >= 0, got {mu}")
    if not 0.0 < delta <= 1.0:
        raise ConfigurationError(f"delta must be in (0, 1], got {delta}")
    if mu == 0.0 or delta >= 1.0 or _gdp_delta(mu, 0.0) <= delta:
        return 0.0
    lo, hi = 0.0, mu * mu + 4.0 * mu
    while _gdp_delta(mu, hi) > delta:
        hi *= 2.0
    for _ in range(100):
        mid = 0.5 * (lo + hi)
        if _gdp_delta(mu, mid) > delta:
            lo = mid
        else:
            hi = mid
        if hi - lo < 1e-12:
            break
    return lo


def _mistake_probabilities(m: int, ranks: int, mu: float, grid_size: int) -> np.ndarray:
    """``v_k`` for the ``ranks`` most confident guesses (k = m-ranks+1 .. m by increasing |privacy loss|)."""
    z = np.linspace(-6.0, mu + 6.0, grid_size)
    mass = 0.5 * (scipy.stats.norm.pdf(z) + scipy.stats.norm.pdf(z - mu)) * (z[1] - z[0])
    loss = np.abs(0.5 * mu * mu - mu * z)
    order = np.argsort(loss, kind="stable")
    mass, loss = mass[order], loss[order]
    cdf = np.concatenate(([0.0], np.cumsum(mass)[:-1]))
    k = np.arange(m - ranks + 1, m + 1, dtype=np.float64)[:, None]
    log_binom = scipy.special.gammaln(m + 1) - scipy.special.gammaln(k) - scipy.special.gammaln(m - k + 1)
    tiny = 1e-300
    log_f = np.where(k > 1, (k - 1) * np.log(np.maximum(cdf, tiny))[None, :], 0.0)
    log_1f = np.where(k < m, (m - k) * np.log(np.maximum(1.0 - cdf, tiny))[None, :], 0.0)
    log_err = scipy.special.log_expit(-loss)[None, :]              # P(wrong | loss) = 1 / (1 + e^{|L|})
    total = log_binom + np.log(np.maximum(mass, tiny))[None, :] + log_f + log_1f + log_err
    return np.clip(np.exp(scipy.special.logsumexp(total, axis=1)), 0.0, 0.5)


def _poisson_binomial_lower_tail(v: np.ndarray, extra: int, v_extra: float, u: int) -> float:
    """Chernoff bound on P(sum of independent Bernoulli(v_k) (+ ``extra`` copies of Bernoulli(v_extra)) <= u)."""
    if u >= float(v.sum()) + extra * v_extra:
        return 1.0
    if u == 0:
        return min(math.exp(float(np.log(np.maximum(1.0 - v, 1e-300)).sum()) + extra * math.log1p(-v_extra)), 1.0)

    def slope(lam):
        e = math.exp(lam)
        return -u + float((v * e / (1.0 + v * (e - 1.0))).sum()) + extra * v_extra * e / (1.0 + v_extra * (e - 1.0))

    lo, hi = -50.0, 0.0
    if slope(lo) >= 0:
        lam = lo
    else:
        for _ in range(100):
            mid = 0.5 * (lo + hi)
            if slope(mid) > 0:
                hi = mid
            else:
                lo = mid
            if hi - lo < 1e-10:
                break
        lam = 0.5 * (lo + hi)
    e = math.exp(lam)
    log_bound = -lam * u + float(np.log1p(v * (e - 1.0)).sum()) + extra * math.log1p(v_extra * (e - 1.0))
    return min(math.exp(log_bound), 1.0)


def _gdp_p_value(m: int, guesses: int, mistakes: int, mu: float, grid_size: int) -> float:
    if not math.isfinite(mu) or mu <= 0.0:
        return 1.0
    exact = min(guesses, 2000)                      # ranks integrated exactly; the rest reuse the weakest of them
    v = _mistake_probabilities(m, exact, mu, grid_size)
    return _poisson_binomial_lower_tail(v, guesses - exact, float(v[0]) if guesses > exact else 0.0, mistakes)


@dataclasses.dataclass(frozen=True)
class GdpMethod:
    _estimate: "OneRunEstimate"
    grid_size: int = 10_000

    def _mu_at(self, significance: float, threshold: float | None) -> float:
        _check_significance(significance)
        m = self._estimate.n_in + self._estimate.n_out
        guesses, wrong = self._estimate._best_r_u(threshold)
        hi = _search_ceiling(m, 0.0, significance)
        for _ in range(60):
            if _gdp_p_value(m, guesses, wrong, hi, self.grid_size) >= significance:
                break
            hi *= 2.0
        else:
            raise OperationError(f"cannot invert mu-GDP p-value for (m={m}, r={guesses}, u={wrong}) at significance="
                                 f"{significance}: p-value stays below it for every mu up to {hi:g}; use fewer canaries "
                                 "or a larger significance.")
        lo = 0.0
        for _ in range(100):
            if hi - lo <= 0.01 * max(1.0, hi):
                break
            mid = 0.5 * (lo + hi)
            if _gdp_p_value(m, guesses, wrong, mid, self.grid_size) < significance:
                lo = mid
            else:
                hi = mid
        return lo

    def epsilon_at(self, *, delta: float, significance: float = 0.05, threshold: float | None = None) -> float:
        if delta <= 0:
            raise ConfigurationError(f"mu-GDP f-DP auditing requires delta > 0, got {delta}")
        _check_delta(delta)
        return _gdp_to_eps(self._mu_at(significance, threshold), delta)

    def delta_at(self, *, epsilon: float, significance: float = 0.05, threshold: float | None = None) -> float:
        if epsilon < 0:
            raise ConfigurationError(f"epsilon must be >= 0, got {epsilon}")
        mu = self._mu_at(significance, threshold)
        return 0.0 if mu == 0.0 else max(0.0, _gdp_delta(mu, epsilon))

    def beta_at(self, *, alpha: float, significance: float = 0.05, threshold: float | None = None) -> float:
        if not 0.0 <= alpha <= 1.0:
            raise ConfigurationError(f"alpha must be in [0, 1], got {alpha}")
        mu = self._mu_at(significance, threshold)
        return float(scipy.stats.norm.cdf(scipy.stats.norm.ppf(1.0 - alpha) - mu))

    def advantage(self, *, significance: float = 0.05, threshold: float | None = None) -> float:
        return float(2.0 * scipy.stats.norm.cdf(self._mu_at(significance, threshold) / 2.0) - 1.0)


# ------------------------------------------------------------------------------------------------ estimate
@dataclasses.dataclass(frozen=True)
class OneRunEstimate:
    n_in: int
    n_out: int
    thresholds: np.ndarray
    tn_counts: np.ndarray
    fn_counts: np.ndarray
    tp_counts: np.ndarray
    fp_counts: np.ndarray
    in_scores: np.ndarray
    out_scores: np.ndarray
    canary_indices: np.ndarray | None = None

    def __repr__(self):
        return f"OneRunEstimate(n_in={self.n_in}, n_out={self.n_out}, auc={_auc(self.tn_counts, self.fn_counts):.4f})"

    def _best_r_u(self, threshold: float | None = None) -> tuple[int, int]:
        """(number of guesses, number of mistakes) at ``threshold``, or at the accuracy-maximising threshold."""
        m = self.n_in + self.n_out
        if threshold is not None:
            right = int(np.sum(self.in_scores >= threshold)) + int(np.sum(self.out_scores < threshold))
            return m, m - right
        return m, m - int(np.max(self.n_in - self.fn_counts + self.tn_counts))

    def eps_delta(self) -> EpsDeltaMethod:
        return EpsDeltaMethod(_estimate=self)

    def gdp(self, *, grid_size: int = 10_000) -> GdpMethod:
        if grid_size < 1000:
            raise ConfigurationError(f"grid_size must be >= 1000, got {grid_size}")
        return GdpMethod(_estimate=self, grid_size=grid_size)

    def epsilon_at(self, *, delta: float, significance: float = 0.05, threshold: float | None = None) -> float:
        return self.gdp().epsilon_at(delta=delta, significance=significance, threshold=threshold)

    def delta_at(self, *, epsilon: float, significance: float = 0.05, threshold: float | None = None) -> float:
        return self.gdp().delta_at(epsilon=epsilon, significance=significance, threshold=threshold)

    def beta_at(self, *, alpha: float, significance: float = 0.05, threshold: float | None = None) -> float:
        return self.gdp().beta_at(alpha=alpha, significance=significance, threshold=threshold)

    def advantage(self, *, significance: float = 0.05, threshold: float | None = None) -> float:
        return self.gdp().advantage(significance=significance, threshold=threshold)

    def attack_auc(self, *, confidence: float | None = None, num_samples: int = 1000, key=None):
        """Area under the attack ROC; with ``confidence`` a bias-corrected bootstrap interval (needs an RNG key)."""
        point = _auc(self.tn_counts, self.fn_counts)
        if confidence is None:
            return point
        if not 0 < confidence < 1:
            raise ConfigurationError(f"confidence must be in (0, 1), got {confidence}")
        if key is None:
            raise ConfigurationError("attack_auc(confidence=...) requires an explicit RNG key for bootstrap resampling")
        rng = np.random.default_rng(seed=key.seed)
        vals = np.empty(num_samples)
        for i in range(num_samples):
            _, tn, fn = get_tn_fn_counts(rng.choice(self.in_scores, size=self.n_in),
                                         rng.choice(self.out_scores, size=self.n_out))
            vals[i] = _auc(tn, fn)
        z0 = scipy.stats.norm.ppf((int(np.sum(vals < point)) + 1) / (num_samples + 2))
        tail = (1 - confidence) / 2
        q = scipy.stats.norm.cdf(2 * z0 + scipy.stats.norm.ppf((tail, 1 - tail)))
        lo, hi = np.quantile(vals, q, method="linear")
        return float(lo), float(hi)

    def attack_beta_at(self, *, alpha):
        return 1.0 - tpr_at_given_fpr(alpha, self.tp_counts, self.fp_counts)


def one_run(scores: CanaryScores, *, coin_flip: CoinFlip) -> OneRunEstimate:
    inside, outside = coin_flip.split_scores(scores)
    if inside.size == 0 or outside.size == 0:
        raise ConfigurationError("Both in_scores and out_scores must be non-empty")
    if not (np.all(np.isfinite(inside)) and np.all(np.isfinite(outside))):
        raise ConfigurationError("scores must contain only finite values")
    thr, tn, fn = get_tn_fn_counts(inside, outside)
    return OneRunEstimate(n_in=len(inside), n_out=len(outside), thresholds=thr, tn_counts=tn, fn_counts=fn,
                          tp_counts=(fn[-1] - fn)[::-1], fp_counts=(tn[-1] - tn)[::-1], in_scores=inside,
                          out_scores=outside, canary_indices=coin_flip.canary_indices)
