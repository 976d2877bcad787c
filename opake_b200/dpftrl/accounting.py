"""DP-FTRL accounting: the matrix-factorisation Gaussian mechanism and its sampling amplifiers
(packages/opake-dpftrl/src/opake/api/accounting/dpftrl/mechanisms/_mf_gaussian.py:44-229,
amplification/_poisson.py:43-222, _balls_in_bins.py:84-254, _b_min_sep/__init__.py:63-207).

* ``MfGaussian``: the whole run is one Gaussian mechanism with multiplier ``nm / sens(C)``.
* ``CyclicPoisson``: with ``bands`` groups, each group sees a Poisson-subsampled banded mechanism
  ``ceil(n_steps / bands)`` times; the groups are disjoint, so the run costs one group's composition.
* ``BallsInBins``: identity strategy -> random allocation / Poisson bound; otherwise the Monte-Carlo estimator over the
  strategy's balls-in-bins Gram matrix.
* ``BMinSep``: accounted without amplification through the min-sep sensitivity (a valid upper bound).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from ..accounting._native import native
from ..accounting.core import DpHorizonProcess, DpProcess
from ..base.exceptions import ConfigurationError, InputTypeError
from ..base.serialization import register_serializer
from .strategies import BandMfStrategy, IdentityStrategy, MfStrategy, deserialize_strategy, serialize_strategy


@dataclass(frozen=True, eq=False)
class MfGaussian(DpProcess):
    noise_multiplier: float
    strategy: MfStrategy
    n_steps: int | None = None
    min_sep: int = 1
    max_participations: int | None = None

    def __post_init__(self):
        if self.noise_multiplier < 0:
            raise ConfigurationError(f"noise_multiplier must be non-negative, got {self.noise_multiplier}")
        if self.n_steps is not None and self.n_steps < 1:
            raise ConfigurationError(f"n_steps must be >= 1, got {self.n_steps}")
        if self.min_sep < 1:
            raise ConfigurationError(f"min_sep must be >= 1, got {self.min_sep}")
        if self.max_participations is not None and self.max_participations < 1:
            raise ConfigurationError(f"max_participations must be >= 1 or None, got {self.max_participations}")

    def _key(self):
        return ("MfGaussian", self.noise_multiplier, self.n_steps, self.min_sep, self.max_participations,
                repr(sorted(serialize_strategy(self.strategy).items(), key=lambda kv: kv[0])))

    def __eq__(self, other):
        return isinstance(other, MfGaussian) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())

    def _pld_cache_key(self):
        return self._key()

    @property
    def _horizon(self) -> int:
        if self.n_steps is None:
            raise ConfigurationError("Bare MfGaussian accounting requires explicit n_steps. Supply the release horizon, or "
                                     "wrap the recipe in a DP-FTRL amplifier.")
        return self.n_steps

    def sensitivity(self) -> float:
        n = self._horizon
        k = self.max_participations if self.max_participations is not None else n
        return self.strategy.sensitivity(n_steps=n, min_sep=self.min_sep, max_participations=k)

    def _build_pld(self, cfg, overrides):
        if self.noise_multiplier == 0:
            return native().non_private_pld(cfg)
        return native().mf_gaussian_pld(float(self.noise_multiplier), float(self.sensitivity()), cfg)


def _save_mf(p: MfGaussian) -> dict[str, Any]:
    return {"type": "MfGaussian", "noise_multiplier": p.noise_multiplier, "strategy": serialize_strategy(p.strategy),
            "n_steps": p.n_steps, "min_sep": p.min_sep, "max_participations": p.max_participations}


def _load_mf(_t, sd) -> MfGaussian:
    return MfGaussian(float(sd["noise_multiplier"]), deserialize_strategy(dict(sd["strategy"])), sd.get("n_steps"),
                      int(sd.get("min_sep", 1)), sd.get("max_participations"))


register_serializer(MfGaussian, _save_mf, _load_mf)


def _inner_ok(inner):
    from ..accounting.core import NonPrivate

    if not isinstance(inner, (MfGaussian, NonPrivate)):
        raise InputTypeError(f"DP-FTRL amplifiers wrap an MfGaussian (or NonPrivate) process, got {type(inner).__name__}.")


@dataclass(frozen=True, eq=False)
class CyclicPoisson(DpHorizonProcess):
    inner: DpProcess
    sample_rate: float
    n_steps: int
    truncated_batch_size: int | None = None
    dataset_size: int | None = None

    def __post_init__(self):
        _inner_ok(self.inner)
        if not 0 < self.sample_rate <= 1:
            raise ConfigurationError(f"sample_rate must be in (0, 1], got {self.sample_rate}")
        if self.n_steps < 1:
            raise ConfigurationError(f"n_steps must be >= 1, got {self.n_steps}")

    def __eq__(self, o):
        return isinstance(o, CyclicPoisson) and self._pld_cache_key() == o._pld_cache_key()

    def __hash__(self):
        return hash(self._pld_cache_key())

    def _pld_cache_key(self):
        return ("CyclicPoisson", self.inner._pld_cache_key() if isinstance(self.inner, MfGaussian) else "np",
                self.sample_rate, self.n_steps, self.truncated_batch_size, self.dataset_size)

    def _build_pld(self, cfg, overrides):
        from ..accounting.core import NonPrivate

        if isinstance(self.inner, NonPrivate) or self.inner.noise_multiplier == 0:
            return native().non_private_pld(cfg)
        strat = self.inner.strategy
        bands = strat.bands if isinstance(strat, BandMfStrategy) else 1
        # one participation inside a band window: sensitivity is the column norm
        c = strat.strategy_coefficients(self.n_steps)
        col = math.sqrt(float((c * c).sum())) if not isinstance(strat, IdentityStrategy) else 1.0
        nm = self.inner.noise_multiplier / col
        if self.truncated_batch_size is not None and self.dataset_size is not None:
            step = native().truncated_poisson_gaussian_pld(nm, self.sample_rate, int(self.truncated_batch_size),
                                                           max(1, int(self.dataset_size) // bands), cfg)
        else:
            base = native().gaussian_pld(nm, cfg)
            step = base if self.sample_rate == 1.0 else native().poisson_pld(base, self.sample_rate, cfg)
        return step.self_compose(math.ceil(self.n_steps / bands))


@dataclass(frozen=True, eq=False)
class BallsInBins(DpHorizonProcess):
    inner: DpProcess
    num_bins: int
    n_steps: int

    def __post_init__(self):
        _inner_ok(self.inner)
        if self.num_bins < 2:
            raise ConfigurationError(f"num_bins must be >= 2, got {self.num_bins}")
        if self.n_steps < 1 or self.n_steps % self.num_bins:
            raise ConfigurationError(f"n_steps ({self.n_steps}) must be a positive multiple of num_bins ({self.num_bins})")

    def __eq__(self, o):
        return isinstance(o, BallsInBins) and self._pld_cache_key() == o._pld_cache_key()

    def __hash__(self):
        return hash(self._pld_cache_key())

    def _pld_cache_key(self):
        return ("BallsInBins", self.inner._pld_cache_key() if isinstance(self.inner, MfGaussian) else "np",
                self.num_bins, self.n_steps)

    def _build_pld(self, cfg, overrides):
        from ..accounting.core import NonPrivate

        if isinstance(self.inner, NonPrivate) or self.inner.noise_multiplier == 0:
            return native().non_private_pld(cfg)
        epochs = self.n_steps // self.num_bins
        strat = self.inner.strategy
        if isinstance(strat, IdentityStrategy):
            return native().balls_in_bins_gaussian_pld_epochs(float(self.inner.noise_multiplier), self.num_bins, epochs, cfg)
        G = strat.gram_matrix(n_steps=self.n_steps, num_bins=self.num_bins, num_epochs=epochs)
        return native().bnb_mc_pld([float(x) for x in G.reshape(-1)], self.num_bins, float(self.inner.noise_multiplier), cfg)


def participation_p_from_per_example_rate(p0: float, bands: int) -> float:
    """Per-step sampling probability of an eligible example such that the stationary participation rate is ``p0``."""
    if not 0 < p0 < 1.0 / bands + 1e-12:
        raise ConfigurationError(f"p0 must be in (0, 1/bands], got {p0}")
    return p0 / (1.0 - (bands - 1) * p0)


@dataclass(frozen=True, eq=False)
class BMinSep(DpHorizonProcess):
    inner: DpProcess
    n_steps: int
    p0: float = 0.0

    def __post_init__(self):
        _inner_ok(self.inner)
        if self.n_steps < 1:
            raise ConfigurationError(f"n_steps must be >= 1, got {self.n_steps}")

    def __eq__(self, o):
        return isinstance(o, BMinSep) and self._pld_cache_key() == o._pld_cache_key()

    def __hash__(self):
        return hash(self._pld_cache_key())

    def _pld_cache_key(self):
        return ("BMinSep", self.inner._pld_cache_key() if isinstance(self.inner, MfGaussian) else "np", self.n_steps, self.p0)

    def _build_pld(self, cfg, overrides):
        from ..accounting.core import NonPrivate

        if isinstance(self.inner, NonPrivate) or self.inner.noise_multiplier == 0:
            return native().non_private_pld(cfg)
        strat = self.inner.strategy
        bands = strat.bands if isinstance(strat, BandMfStrategy) else 1
        coef = [float(x) for x in strat.strategy_coefficients(self.n_steps)]
        p = participation_p_from_per_example_rate(self.p0, bands) if self.p0 else 1.0
        return native().bandmf_b_min_sep_warm_mc_pld(coef, self.n_steps, min(1.0, p), float(self.inner.noise_multiplier), cfg)


def mf_gaussian(noise_multiplier: float, strategy: MfStrategy, *, n_steps: int | None = None, min_sep: int = 1,
                max_participations: int | None = None) -> MfGaussian:
    return MfGaussian(noise_multiplier, strategy, n_steps, min_sep, max_participations)


def poisson(inner, sample_rate: float, *, n_steps: int, truncated_batch_size: int | None = None,
            dataset_size: int | None = None) -> CyclicPoisson:
    return CyclicPoisson(inner, sample_rate, n_steps, truncated_batch_size, dataset_size)


def balls_in_bins(inner, *, num_bins: int, n_steps: int) -> BallsInBins:
    return BallsInBins(inner, num_bins, n_steps)


def b_min_sep(inner, *, n_steps: int, p0: float) -> BMinSep:
    return BMinSep(inner, n_steps, p0)


__all__ = ["MfGaussian", "CyclicPoisson", "BallsInBins", "BMinSep", "mf_gaussian", "poisson", "balls_in_bins", "b_min_sep",
           "participation_p_from_per_example_rate"]
