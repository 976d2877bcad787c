"""How one noise multiplier is spread over parameter groups and over paired (first/second moment) streams.

Formulas as in packages/opake-engine/src/opake/api/engine/noise_allocation.py:40-287:
``sigma_g = nm * sqrt(C_g * sum_h C_h)`` (MSE-optimal under the Mahalanobis constraint, accounted as one
``gaussian(nm)``); paired release ``S = sum(D1 + D2)``, ``sigma = nm * sqrt(D * S)`` per stream and group.
"""
from __future__ import annotations

import math

from ..base.exceptions import ConfigurationError, InputTypeError
from .types import ClippedPytree, PerGroup, SecondMomentClippingOutput

PAIRED_FIRST_STREAM_FOLD = "opake.paired.first"
PAIRED_SECOND_STREAM_FOLD = "opake.paired.second"


def per_group_noise_stddev(max_norm: PerGroup, noise_multiplier: float) -> PerGroup:
    if not isinstance(max_norm, PerGroup):
        raise InputTypeError(f"per_group_noise_stddev requires a PerGroup max_norm, got {type(max_norm).__name__}.")
    if noise_multiplier < 0:
        raise ConfigurationError(f"noise_multiplier must be non-negative, got {noise_multiplier}")
    for g, v in max_norm.values.items():
        if v < 0:
            raise ConfigurationError(f"per-group bounds must be non-negative, got {v} for group '{g}'.")
    if noise_multiplier == 0.0:
        return PerGroup(max_norm.groups, dict.fromkeys(max_norm.values, 0.0))
    total = sum(max_norm.values.values())
    return PerGroup(max_norm.groups, {k: noise_multiplier * math.sqrt(c * total) for k, c in max_norm.values.items()})


def _check(value, label: str) -> None:
    if isinstance(value, PerGroup):
        for n, v in value.values.items():
            if v < 0:
                raise ConfigurationError(f"{label} per-group bounds must be non-negative, got {v} for group '{n}'.")
        return
    if not isinstance(value, (int, float)):
        raise InputTypeError(f"{label} must be float or PerGroup, got {type(value).__name__}.")
    if value < 0:
        raise ConfigurationError(f"{label} must be non-negative, got {value}.")


def _total(value) -> float:
    return float(sum(value.values.values())) if isinstance(value, PerGroup) else float(value)


def _sigma(value, total: float, nm: float):
    if isinstance(value, PerGroup):
        return PerGroup(value.groups, {k: nm * math.sqrt(v * total) for k, v in value.values.items()})
    return nm * math.sqrt(float(value) * total)


def paired_noise_stddevs(noise_multiplier: float, *, first, second):
    """Joint allocation for releasing both moment streams with the PLD of a single ``gaussian(nm)``."""
    if isinstance(first, PerGroup) != isinstance(second, PerGroup):
        raise InputTypeError("paired_noise_stddevs requires both streams to have the same kind; got "
                             f"first={type(first).__name__}, second={type(second).__name__}.")
    if noise_multiplier < 0:
        raise ConfigurationError(f"noise_multiplier must be non-negative, got {noise_multiplier}")
    _check(first, "first")
    _check(second, "second")
    if isinstance(first, PerGroup):
        if first.groups != second.groups:
            raise ConfigurationError("paired_noise_stddevs requires identical group mappings on both streams; got "
                                     f"{len(first.groups)} vs {len(second.groups)} parameter assignments.")
        if set(first.values) != set(second.values):
            raise ConfigurationError("paired_noise_stddevs requires identical group sets on both streams; got "
                                     f"{sorted(first.values)} vs {sorted(second.values)}.")
    total = _total(first) + _total(second)
    return _sigma(first, total, noise_multiplier), _sigma(second, total, noise_multiplier)


def resolve_paired_clipped(clipped_input: SecondMomentClippingOutput, *, noise_multiplier: float):
    a, b = clipped_input.grads, clipped_input.squared_grads
    if not isinstance(a, ClippedPytree):
        raise InputTypeError("SecondMomentClippingOutput.grads must be a ClippedPytree.")
    if not isinstance(b, ClippedPytree):
        raise InputTypeError("SecondMomentClippingOutput.squared_grads must be a ClippedPytree.")
    s1, s2 = paired_noise_stddevs(noise_multiplier, first=a.max_norm, second=b.max_norm)
    return a, b, s1, s2


__all__ = ["PAIRED_FIRST_STREAM_FOLD", "PAIRED_SECOND_STREAM_FOLD", "paired_noise_stddevs", "per_group_noise_stddev",
           "resolve_paired_clipped"]
