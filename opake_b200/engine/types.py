"""DP-aware pytree wrappers: sensitivity travels with the clipped value, noise scale with the noised value.

Semantics follow packages/opake-engine/src/opake/api/engine/types.py:71-477: ``PerGroup`` (per-parameter-group
scalars with ``effective = sqrt(sum v^2)``), ``ClippedPytree`` (only public-scalar ``*``, ``/`` and negation keep the
clipped interpretation; ``+``/``-``/``**`` raise), ``NoisedPytree`` (adds the realised noise stddev), and the paired
first/second-moment containers.
"""
from __future__ import annotations

import math
from abc import ABC
from collections.abc import Mapping
from dataclasses import dataclass, replace
from numbers import Real
from types import MappingProxyType
from typing import Any, Literal, NamedTuple

import torch

from ..base.exceptions import ConfigurationError, InputTypeError
from .pytree import ParamPath, param_path, tree_map
from .random import RngKey

TensorPytree = Any
MaxNorm = Any
NoiseStddev = Any


@dataclass(frozen=True)
class PerGroup:
    """One scalar per named parameter group plus the leaf-path -> group assignment."""

    groups: Mapping
    values: Mapping

    def __post_init__(self) -> None:
        object.__setattr__(self, "groups", MappingProxyType({param_path(k): g for k, g in self.groups.items()}))
        object.__setattr__(self, "values", MappingProxyType(dict(self.values)))

    @property
    def effective(self) -> float:
        return math.sqrt(sum(v * v for v in self.values.values()))

    @property
    def num_groups(self) -> int:
        return len(self.values)

    def _map(self, fn) -> "PerGroup":
        return PerGroup(self.groups, {k: fn(k, v) for k, v in self.values.items()})

    def __rmul__(self, scalar: float) -> "PerGroup":
        return self._map(lambda _k, v: scalar * v)

    def __mul__(self, other) -> "PerGroup":
        if isinstance(other, PerGroup):
            if other.groups != self.groups:
                raise ConfigurationError("PerGroup × PerGroup requires identical group mappings; got groups with "
                                         f"{len(self.groups)} vs {len(other.groups)} parameter assignments.")
            if set(other.values) != set(self.values):
                raise ConfigurationError("PerGroup × PerGroup requires identical group sets; got "
                                         f"{sorted(self.values)} vs {sorted(other.values)}.")
            return self._map(lambda k, v: v * other.values[k])
        return self._map(lambda _k, v: v * other)

    def __truediv__(self, scalar: float) -> "PerGroup":
        return self._map(lambda _k, v: v / scalar)

    def for_path(self, path) -> float:
        return self.values[self.groups[param_path(path)]]

    def __hash__(self):
        return hash((tuple(sorted(self.values.items())), len(self.groups)))


class ClipState(ABC):  # noqa: B024
    """Marker base of the explicit state token returned by clipping transforms."""


class NoiseState(ABC):  # noqa: B024
    """Base of noise-mechanism states (``_step_counter`` calls made, immutable ``_rng_key``)."""

    _step_counter: int
    _rng_key: RngKey


def _public_scalar(x: Any, op: str) -> float:
    if isinstance(x, bool) or not isinstance(x, Real):
        raise InputTypeError(f"{op} only supports public real-number scalars. Operate on `.pytree` and reconstruct the "
                             "clipped value with an explicit max_norm when the clipped interpretation is unclear.")
    return float(x)


def _map_tensors(tree: Any, fn) -> Any:
    return tree_map(lambda leaf: fn(leaf) if isinstance(leaf, torch.Tensor) else leaf, tree)


def _refuse(op: str):
    return InputTypeError(f"ClippedPytree {op} does not preserve DP max_norm semantics automatically. Operate on "
                          "`.pytree` and reconstruct the clipped value with an explicit max_norm.")


@dataclass(frozen=True)
class ClippedPytree:
    """A pytree whose dependence on any single record is bounded in L2 by ``max_norm``."""

    pytree: Any
    max_norm: MaxNorm

    @property
    def sensitivity(self) -> float:
        eff = getattr(self.max_norm, "effective", None)
        return float(eff if eff is not None else self.max_norm)

    def noise_stddev_for(self, *, noise_multiplier: float, allocation: Literal["isotropic", "optimal"] = "optimal"):
        if noise_multiplier < 0:
            raise ConfigurationError(f"noise_multiplier must be non-negative, got {noise_multiplier}")
        if allocation not in ("isotropic", "optimal"):
            raise ConfigurationError(f"allocation must be 'isotropic' or 'optimal', got {allocation!r}.")
        if isinstance(self.max_norm, PerGroup):
            if allocation == "isotropic":
                return noise_multiplier * self.max_norm.effective
            from .noise_allocation import per_group_noise_stddev

            return per_group_noise_stddev(self.max_norm, noise_multiplier)
        return noise_multiplier * float(self.max_norm)

    def _scaled(self, c: float):
        return replace(self, pytree=_map_tensors(self.pytree, lambda t: t * c), max_norm=abs(c) * self.max_norm)

    def __mul__(self, s):
        return self._scaled(_public_scalar(s, "ClippedPytree *"))

    def __rmul__(self, s):
        return self._scaled(_public_scalar(s, "* ClippedPytree"))

    def __truediv__(self, s):
        f = _public_scalar(s, "ClippedPytree /")
        if f == 0.0:
            raise ZeroDivisionError("ClippedPytree division by zero")
        return self._scaled(1.0 / f)

    def __rtruediv__(self, s):
        raise _refuse("reverse division")

    def __neg__(self):
        return self._scaled(-1.0)

    def __add__(self, o):
        raise _refuse("addition")

    __radd__ = __add__

    def __sub__(self, o):
        raise _refuse("subtraction")

    __rsub__ = __sub__

    def __pow__(self, e):
        raise _refuse("power")

    def clone(self):
        return replace(self, pytree=_map_tensors(self.pytree, lambda t: t.clone()))

    def detach(self):
        return replace(self, pytree=_map_tensors(self.pytree, lambda t: t.detach()))

    def to(self, *a, **k):
        return replace(self, pytree=_map_tensors(self.pytree, lambda t: t.to(*a, **k)))


@dataclass(frozen=True)
class NoisedPytree(ClippedPytree):
    """A privatised pytree: ``max_norm`` is still the record-impact bound, ``noise_stddev`` the realised noise."""

    noise_stddev: NoiseStddev = None

    def _scaled(self, c: float):
        sd = None if self.noise_stddev is None else abs(c) * self.noise_stddev
        return replace(self, pytree=_map_tensors(self.pytree, lambda t: t * c), max_norm=abs(c) * self.max_norm,
                       noise_stddev=sd)


class SecondMomentClippingOutput(NamedTuple):
    """Pre-noise pair: clipped ``sum g_i`` and clipped ``sum g_i^2`` (squared per example inside the clip loop)."""

    grads: ClippedPytree
    squared_grads: ClippedPytree


class SecondMomentNoiseOutput(NamedTuple):
    """Post-noise pair for optimizers with a private second-moment stream."""

    noisy_grads: NoisedPytree
    noisy_squared_grads: NoisedPytree


def clipped(pytree: Any, *, max_norm: MaxNorm) -> ClippedPytree:
    return ClippedPytree(pytree=pytree, max_norm=max_norm)


def noised(pytree: Any, *, max_norm: MaxNorm, noise_stddev: NoiseStddev) -> NoisedPytree:
    return NoisedPytree(pytree=pytree, max_norm=max_norm, noise_stddev=noise_stddev)


__all__ = ["ClipState", "ClippedPytree", "MaxNorm", "NoiseState", "NoiseStddev", "NoisedPytree", "ParamPath", "PerGroup",
           "SecondMomentClippingOutput", "SecondMomentNoiseOutput", "TensorPytree", "clipped", "noised"]
