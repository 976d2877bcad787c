"""DP-FTRL glue of the trainer (packages/opake-transformers/src/opake/api/transformers/trainer/
_dpftrl.py:55-398): builds the matrix-factorisation strategy named by ``privacy_noise_mechanism``, the matching
amplification accounting, and the sampler that the analysis assumes."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable

from .. import dpftrl as F
from ..base.exceptions import ConfigurationError
from ..dpftrl import accounting as FA
from ..dpftrl import sampling as FS
from ..dpsgd import accounting as SA
from ..dpsgd import sampling as SS

__all__ = ["MFContext", "build_strategy", "build_amplifier_factory", "build_sampler", "cyclic_poisson_group_rate"]


@dataclass(frozen=True)
class MFContext:
    """Quantities shared by strategy, accounting and sampler of one matrix-factorisation run."""
    n_steps: int
    min_sep: int
    max_participations: int
    bands: int = 1


def build_strategy(kind: str, kwargs: dict, *, lr_schedule=None):
    kw = dict(kwargs)
    if kind == "mf_identity":
        return F.identity_strategy()
    if kind == "mf_band":
        return F.band_mf_strategy(bands=int(kw.pop("bands", 16)), momentum=float(kw.pop("momentum", 1.0)), lr_schedule=lr_schedule)
    if kind == "mf_blt":
        return F.blt_strategy(max_buffers=int(kw.pop("max_buffers", 10)), momentum=float(kw.pop("momentum", 1.0)),
                              lr_schedule=lr_schedule)
    if kind == "mf_bisr":
        return F.bisr_strategy(bandwidth=int(kw.pop("bandwidth", 4)), normalized=bool(kw.pop("normalized", True)),
                               momentum=float(kw.pop("momentum", 0.0)), lr_schedule=lr_schedule)
    if kind == "mf_bsr":
        return F.bsr_strategy(bandwidth=int(kw.pop("bandwidth", 8)), alpha=float(kw.pop("alpha", 1.0)), beta=float(kw.pop("beta", 0.9)))
    if kind == "mf_lambda_cgd":
        return F.lambda_cgd_strategy(lambda_=float(kw.pop("lambda_", 0.5)), normalized=bool(kw.pop("normalized", True)),
                                     lr_schedule=lr_schedule)
    raise ConfigurationError(f"{kind!r} is not a matrix-factorisation mechanism")


def mf_context(kind: str, kwargs: dict, sampling: str, sampling_kwargs: dict, *, n_steps: int, steps_per_epoch: int) -> MFContext:
    bands = int(kwargs.get("bands", 1)) if kind == "mf_band" else 1
    if sampling in ("cyclic_poisson", "b_min_sep"):
        min_sep = bands
    elif sampling == "balls_in_bins":
        min_sep = int(sampling_kwargs.get("num_bins", steps_per_epoch))
    else:
        min_sep = 1
    max_part = int(math.ceil(n_steps / max(1, min_sep)))
    return MFContext(n_steps=n_steps, min_sep=max(1, min_sep), max_participations=max(1, max_part), bands=bands)


def cyclic_poisson_group_rate(sample_rate: float, bands: int) -> float:
    """Within its own group (one of ``bands`` equal parts, visited every ``bands`` steps) an example is drawn with
    ``bands`` times the overall rate so that the expected batch size stays ``sample_rate * N``."""
    q = sample_rate * bands
    if not 0 < q <= 1:
        raise ConfigurationError(f"sample_rate * bands = {q} must be in (0, 1]; lower the batch size or the band count")
    return q


def build_amplifier_factory(kind: str, sampling: str, *, strategy, ctx: MFContext | None, sample_rate: float,
                            dataset_size: int, n_steps: int, sampling_kwargs: dict) -> Callable[[float], Any]:
    """Returns ``noise_multiplier -> DpProcess`` for the whole run (or one step for plain Poisson DP-SGD, where the
    caller repeats it)."""
    trunc = sampling_kwargs.get("truncated_batch_size")
    if kind == "gaussian":
        if sampling == "poisson":
            return lambda nm: SA.poisson(SA.gaussian(nm), sample_rate, truncated_batch_size=trunc, dataset_size=dataset_size if trunc else None)
        if sampling == "k_out_of_t":
            k, t = int(sampling_kwargs["k"]), int(sampling_kwargs["t"])
            return lambda nm: SA.k_out_of_t(SA.gaussian(nm), k=k, t=t, allocation=sampling_kwargs.get("allocation", "random"))
    assert ctx is not None
    if kind == "mf_identity" and sampling == "poisson":
        return lambda nm: SA.poisson(SA.gaussian(nm), sample_rate, truncated_batch_size=trunc, dataset_size=dataset_size if trunc else None)

    def inner(nm):
        return FA.mf_gaussian(nm, strategy, n_steps=ctx.n_steps, min_sep=ctx.min_sep, max_participations=ctx.max_participations)

    if sampling == "cyclic_poisson":
        q = cyclic_poisson_group_rate(sample_rate, ctx.bands)
        return lambda nm: FA.poisson(inner(nm), q, n_steps=ctx.n_steps, truncated_batch_size=trunc, dataset_size=dataset_size if trunc else None)
    if sampling == "balls_in_bins":
        bins = int(sampling_kwargs.get("num_bins", ctx.min_sep))
        return lambda nm: FA.balls_in_bins(inner(nm), num_bins=bins, n_steps=ctx.n_steps)
    if sampling == "b_min_sep":
        p0 = float(sampling_kwargs.get("sampling_prob", cyclic_poisson_group_rate(sample_rate, ctx.bands)))
        return lambda nm: FA.b_min_sep(inner(nm), n_steps=ctx.n_steps, p0=p0)
    raise ConfigurationError(f"no accounting for mechanism {kind!r} with sampling {sampling!r}")


def build_sampler(sampling: str, dataset, *, sample_rate: float, n_steps: int, key, ctx: MFContext | None, sampling_kwargs: dict):
    trunc = sampling_kwargs.get("truncated_batch_size")
    if sampling == "poisson":
        return SS.PoissonSampler(dataset, sample_rate, n_steps=n_steps, truncated_batch_size=trunc, key=key)
    if sampling == "k_out_of_t":
        return SS.KOutOfTSampler(dataset, k=int(sampling_kwargs["k"]), t=int(sampling_kwargs["t"]),
                                 allocation=sampling_kwargs.get("allocation", "random"), key=key)
    assert ctx is not None
    if sampling == "cyclic_poisson":
        return FS.CyclicPoissonSampler(dataset, cyclic_poisson_group_rate(sample_rate, ctx.bands), bands=ctx.bands, n_steps=n_steps,
                                       truncated_batch_size=trunc, key=key)
    if sampling == "balls_in_bins":
        return FS.BallsInBinsSampler(dataset, int(sampling_kwargs.get("num_bins", ctx.min_sep)), n_steps=n_steps, key=key)
    if sampling == "b_min_sep":
        p0 = float(sampling_kwargs.get("sampling_prob", cyclic_poisson_group_rate(sample_rate, ctx.bands)))
        return FS.BMinSepSampler(dataset, ctx.bands, p0, n_steps, key=key)
    raise ConfigurationError(f"unknown sampling mode {sampling!r}")
