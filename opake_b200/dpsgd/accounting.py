"""DP-SGD accounting processes: Gaussian mechanism, adaptive-clipping adjustment, Poisson / parallel Poisson /
k-out-of-t amplification (packages/opake-dpsgd/src/opake/api/accounting/dpsgd/mechanisms/_gaussian.py:17-85,
_adaclip.py:26-144, amplification/_poisson.py:19-222, _parallel_poisson.py:17-143, _k_out_of_t.py:32-143).

Field names are part of the ``accountant.json`` format. Effective noise multipliers:
``AdaClip``: ``1 / sqrt(1/z^2 + K / (4 sigma_b^2))`` with ``sigma_b = fraction_noise_std * expected_batch_size``.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..accounting._native import native
from ..accounting.core import DpHorizonProcess, DpProcess, NonPrivate
from ..base.exceptions import ConfigurationError, InputTypeError


@dataclass(frozen=True)
class Gaussian(DpProcess):
    noise_multiplier: float

    def __post_init__(self):
        nm = float(self.noise_multiplier)
        if not nm >= 0:
            raise ConfigurationError(f"noise_multiplier must be non-negative, got {self.noise_multiplier}")
        object.__setattr__(self, "noise_multiplier", nm)

    @property
    def effective_noise_multiplier(self) -> float:
        return self.noise_multiplier

    def _build_pld(self, cfg, overrides):
        if self.noise_multiplier < native().MIN_NOISE_MULTIPLIER:
            return native().non_private_pld(cfg)
        return native().gaussian_pld(self.noise_multiplier, cfg)


@dataclass(frozen=True)
class AdaClip(DpProcess):
    inner: DpProcess
    fraction_noise_std: float
    expected_batch_size: float
    num_groups: int = 1

    def __post_init__(self):
        if not isinstance(self.inner, (Gaussian, NonPrivate)):
            raise InputTypeError(f"AdaClip requires a Gaussian or NonPrivate inner mechanism, got {type(self.inner).__name__}.")
        if self.fraction_noise_std <= 0 or self.expected_batch_size <= 0 or self.num_groups < 1:
            raise ConfigurationError("fraction_noise_std and expected_batch_size must be > 0 and num_groups >= 1")

    @property
    def effective_noise_multiplier(self) -> float:
        if isinstance(self.inner, NonPrivate) or self.inner.noise_multiplier == 0:
            return 0.0
        sigma_b = self.expected_batch_size * self.fraction_noise_std
        return 1.0 / native().adaclip_sensitivity(self.inner.noise_multiplier, sigma_b, self.num_groups)

    def _build_pld(self, cfg, overrides):
        nm = self.effective_noise_multiplier
        return native().non_private_pld(cfg) if nm < native().MIN_NOISE_MULTIPLIER else native().gaussian_pld(nm, cfg)


def _nm_of(inner) -> float:
    if isinstance(inner, NonPrivate):
        return 0.0
    return float(inner.effective_noise_multiplier)


@dataclass(frozen=True)
class Poisson(DpProcess):
    inner: DpProcess
    sample_rate: float
    truncated_batch_size: int | None = None
    dataset_size: int | None = None

    def __post_init__(self):
        if not isinstance(self.inner, (Gaussian, AdaClip, NonPrivate)):
            raise InputTypeError("Poisson requires a Gaussian, AdaClip, or NonPrivate inner mechanism, got "
                                 f"{type(self.inner).__name__}.")
        q = float(self.sample_rate)
        if not 0 < q <= 1:
            raise ConfigurationError(f"sample_rate must be in (0, 1], got {self.sample_rate}. For q=1 (every example "
                                     "participates) there is no Poisson amplification.")
        object.__setattr__(self, "sample_rate", q)
        if q == 1.0 and self.truncated_batch_size is not None:
            raise ConfigurationError("Poisson: sample_rate=1.0 requires plain Poisson (truncated_batch_size=None).")
        if (self.truncated_batch_size is None) != (self.dataset_size is None):
            raise ConfigurationError("Poisson: truncated_batch_size and dataset_size must be set together (both None for "
                                     "plain Poisson, both set for truncated).")
        if self.truncated_batch_size is not None:
            if type(self.truncated_batch_size) is not int or type(self.dataset_size) is not int:
                raise InputTypeError("truncated_batch_size and dataset_size must be ints")
            if self.truncated_batch_size < 1 or self.dataset_size < 1:
                raise ConfigurationError("truncated_batch_size and dataset_size must be >= 1")

    def _build_pld(self, cfg, overrides):
        nm = _nm_of(self.inner)
        if nm < native().MIN_NOISE_MULTIPLIER:
            return native().non_private_pld(cfg)
        if self.truncated_batch_size is not None:
            return native().truncated_poisson_gaussian_pld(nm, self.sample_rate, self.truncated_batch_size,
                                                           self.dataset_size, cfg)
        base = native().gaussian_pld(nm, cfg)
        return base if self.sample_rate == 1.0 else native().poisson_pld(base, self.sample_rate, cfg)


@dataclass(frozen=True)
class ParallelPoisson(DpProcess):
    inner: Poisson
    num_workers: int

    def __post_init__(self):
        if not isinstance(self.inner, Poisson):
            raise InputTypeError(f"ParallelPoisson requires a Poisson inner process, got {type(self.inner).__name__}.")
        if self.inner.truncated_batch_size is not None:
            raise ConfigurationError("ParallelPoisson does not support truncated Poisson sampling")
        if type(self.num_workers) is not int or self.num_workers < 1:
            raise ConfigurationError(f"num_workers must be a positive int, got {self.num_workers}")

    def _build_pld(self, cfg, overrides):
        nm = _nm_of(self.inner.inner)
        if nm < native().MIN_NOISE_MULTIPLIER:
            return native().non_private_pld(cfg)
        return native().parallel_poisson_gaussian_pld(nm, self.inner.sample_rate, self.num_workers, cfg)


@dataclass(frozen=True)
class KOutOfT(DpHorizonProcess):
    """Whole-horizon process: every record takes part in ``k`` of ``n_steps`` steps ("total" is bounded by "block")."""

    inner: DpProcess
    k: int
    n_steps: int
    allocation: str

    def __post_init__(self):
        if not isinstance(self.inner, (Gaussian, AdaClip, NonPrivate)):
            raise InputTypeError("KOutOfT requires a Gaussian, AdaClip, or NonPrivate inner mechanism")
        if self.n_steps < 1 or not 1 <= self.k <= self.n_steps:
            raise ConfigurationError(f"need n_steps >= 1 and k in [1, n_steps], got k={self.k}, n_steps={self.n_steps}")
        if self.allocation not in ("block", "total"):
            raise ConfigurationError(f"allocation must be 'block' or 'total', got {self.allocation!r}")

    def _build_pld(self, cfg, overrides):
        nm = _nm_of(self.inner)
        if nm < native().MIN_NOISE_MULTIPLIER:
            return native().non_private_pld(cfg)
        return native().random_allocation_gaussian_pld(nm, self.n_steps, self.k, cfg)


def gaussian(noise_multiplier: float) -> Gaussian:
    return Gaussian(noise_multiplier)


def adaclip(inner, *, fraction_noise_std: float = 0.05, expected_batch_size: float, num_groups: int = 1) -> AdaClip:
    return AdaClip(inner, fraction_noise_std, expected_batch_size, num_groups)


def poisson(inner, sample_rate: float, *, truncated_batch_size: int | None = None, dataset_size: int | None = None):
    return Poisson(inner, sample_rate, truncated_batch_size, dataset_size)


def parallel_poisson(inner, sample_rate: float, num_workers: int) -> ParallelPoisson:
    return ParallelPoisson(Poisson(inner, sample_rate), num_workers)


def k_out_of_t(inner, *, k: int, t: int, allocation: str) -> KOutOfT:
    return KOutOfT(inner, k, t, allocation)


__all__ = ["AdaClip", "Gaussian", "KOutOfT", "ParallelPoisson", "Poisson", "adaclip", "gaussian", "k_out_of_t",
           "parallel_poisson", "poisson"]
