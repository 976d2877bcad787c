"""Process algebra of the accountant: ``step * 1000``, ``a | b``, lazily evaluated through the native PLD engine.

Objects and operator rules follow packages/opake-accounting/src/opake/api/accounting/core/_base.py:112-515 and
composition/: every process is a frozen dataclass with ``pld(**overrides)``; ``*`` builds ``Repeated`` (nested
repeats flatten), ``|`` builds ``Composed`` with identity elision and merging of equal steps into ``Repeated``
(also along the right spine, so an accountant that is fed the same step every iteration stays O(1) in size);
subclasses register themselves by class name for the ``{"type": ...}`` JSON codec.
"""
from __future__ import annotations

import dataclasses
import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, ClassVar

from ..base.exceptions import ConfigurationError
from .discretization import OVERRIDE_NAMES, get_discretization

_PROCESS_REGISTRY: dict[str, type] = {}
_PLD_CACHE: "OrderedDict[Any, Any]" = OrderedDict()
_PLD_CACHE_SIZE = 64


def _freeze(v: Any):
    if isinstance(v, DpProcess):
        return v._pld_cache_key()
    if isinstance(v, (list, tuple)):
        return tuple(_freeze(x) for x in v)
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    try:
        hash(v)
        return v
    except TypeError:
        return repr(v)


def cached_pld(proc: "DpProcess", overrides: dict, build):
    cfg = get_discretization(**overrides)
    key = (proc._pld_cache_key(), cfg._key())
    hit = _PLD_CACHE.get(key)
    if hit is not None:
        _PLD_CACHE.move_to_end(key)
        return hit
    out = build(cfg)
    _PLD_CACHE[key] = out
    while len(_PLD_CACHE) > _PLD_CACHE_SIZE:
        _PLD_CACHE.popitem(last=False)
    return out


def clear_pld_cache() -> None:
    _PLD_CACHE.clear()


class DpProcess:
    """A differentially private release (or a composition of releases) whose PLD can be computed on demand."""

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        _PROCESS_REGISTRY[cls.__name__] = cls

    # ---- to implement
    def _build_pld(self, cfg, overrides: dict):
        raise NotImplementedError

    # ---- evaluation
    def pld(self, **overrides):
        bad = set(overrides) - set(OVERRIDE_NAMES)
        if bad:
            raise ConfigurationError(f"unknown discretization overrides: {sorted(bad)}")
        return cached_pld(self, overrides, lambda cfg: self._build_pld(cfg, overrides))

    def epsilon_at(self, delta: float, **overrides) -> float:
        res = get_discretization(mc_resolution=overrides.get("mc_resolution")).mc_resolution
        overrides = dict(overrides, mc_resolution=min(res, delta / 2.0) if delta > 0 else res)
        return self.pld(**overrides).epsilon_at(delta)

    def delta_at(self, epsilon: float, **overrides) -> float:
        return self.pld(**overrides).delta_at(epsilon)

    def advantage(self, **overrides) -> float:
        return self.pld(**overrides).advantage()

    def beta_at(self, alpha: float, **overrides) -> float:
        return self.pld(**overrides).beta_at(alpha)

    def risk_at(self, prior: float, **overrides) -> float:
        return self.pld(**overrides).risk_at(prior)

    def repeated_pld(self, count: int, **overrides):
        """PLD of ``count`` independent applications (mechanisms whose K-fold release is not a K-fold composition
        of the single release override this)."""
        res = get_discretization(mc_resolution=overrides.get("mc_resolution")).mc_resolution
        per = -math.expm1(math.log1p(-res) / count)
        return self.pld(**dict(overrides, mc_resolution=per)).self_compose(count)

    # ---- structure
    def _leaf_and_count(self):
        return self, 1

    def _pld_cache_key(self):
        return (type(self).__name__, tuple(_freeze(getattr(self, f.name)) for f in dataclasses.fields(self)))

    def __mul__(self, count: int) -> "DpProcess":
        if not isinstance(count, int) or isinstance(count, bool) or count < 1:
            raise ConfigurationError(f"Repeat count must be >= 1, got {count}. Use identity() for zero privacy loss.")
        leaf, n = self._leaf_and_count()
        return Repeated(leaf, n * count)

    __rmul__ = __mul__

    def __or__(self, other: "DpProcess") -> "DpProcess":
        if not isinstance(other, DpProcess):
            return NotImplemented
        if isinstance(self, Identity):
            return other
        if isinstance(other, Identity):
            return self
        la, na = self._leaf_and_count()
        lb, nb = other._leaf_and_count()
        if not isinstance(self, Composed) and not isinstance(other, Composed) and la == lb:
            return Repeated(la, na + nb)
        if isinstance(self, Composed) and not isinstance(other, Composed):
            lr, nr = self.right._leaf_and_count()
            if not isinstance(self.right, Composed) and lr == lb:
                return Composed(self.left, Repeated(lr, nr + nb))
        return Composed(self, other)


@dataclass(frozen=True)
class Repeated(DpProcess):
    inner: DpProcess
    count: int

    def __post_init__(self):
        if self.count < 1:
            raise ConfigurationError(f"Repeat count must be >= 1, got {self.count}")

    def _leaf_and_count(self):
        return self.inner, self.count

    def _build_pld(self, cfg, overrides):
        return self.inner.repeated_pld(self.count, **overrides)


@dataclass(frozen=True, eq=False)
class Composed(DpProcess):
    left: DpProcess
    right: DpProcess

    def _flatten(self) -> list[DpProcess]:
        out, stack = [], [self]
        while stack:
            n = stack.pop()
            if isinstance(n, Composed):
                stack.append(n.right)
                stack.append(n.left)
            else:
                out.append(n)
        return out

    def __eq__(self, other):
        return isinstance(other, Composed) and self._flatten() == other._flatten()

    def __hash__(self):
        return hash(tuple(hash(x) for x in self._flatten()))

    def __repr__(self):
        return "Composed(" + " | ".join(repr(x) for x in self._flatten()) + ")"

    def _pld_cache_key(self):
        return ("Composed", tuple(x._pld_cache_key() for x in self._flatten()))

    def _build_pld(self, cfg, overrides):
        parts = self._flatten()
        out = parts[0].pld(**overrides)
        for p in parts[1:]:
            out = out.compose(p.pld(**overrides))
        return out


@dataclass(frozen=True)
class CachedProcess(DpProcess):
    """Merge barrier: keeps ``inner`` as one node (its PLD is cached as a unit)."""

    inner: DpProcess
    maxsize: int = 8

    def _pld_cache_key(self):
        return ("CachedProcess", self.inner._pld_cache_key())

    def _build_pld(self, cfg, overrides):
        return self.inner.pld(**overrides)


@dataclass(frozen=True)
class EpsDelta(DpProcess):
    epsilon: float
    delta: float = 0.0

    def __post_init__(self):
        if self.epsilon < 0 or not 0 <= self.delta <= 1:
            raise ConfigurationError(f"need epsilon >= 0 and delta in [0, 1], got ({self.epsilon}, {self.delta})")

    def _build_pld(self, cfg, overrides):
        from ._native import native

        return native().eps_delta_pld(float(self.epsilon), float(self.delta), cfg)


@dataclass(frozen=True)
class Identity(DpProcess):
    def _build_pld(self, cfg, overrides):
        from ._native import native

        return native().identity_pld(cfg)


@dataclass(frozen=True)
class NonPrivate(DpProcess):
    def _build_pld(self, cfg, overrides):
        from ._native import native

        return native().non_private_pld(cfg)


class DpHorizonProcess(DpProcess):
    """A process that covers a whole pre-declared training horizon (DP-FTRL); it cannot be extended step by step."""

    is_horizon: ClassVar[bool] = True


def repeat(process: DpProcess, count: int) -> DpProcess:
    return process * count


def compose(*processes: DpProcess) -> DpProcess:
    out: DpProcess = Identity()
    for p in processes:
        out = out | p
    return out


def cached(process: DpProcess, maxsize: int = 8) -> DpProcess:
    return CachedProcess(process, maxsize)


def eps_delta(epsilon: float, delta: float = 0.0) -> DpProcess:
    return EpsDelta(epsilon, delta)


def identity() -> DpProcess:
    return Identity()


def nonprivate() -> DpProcess:
    return NonPrivate()


__all__ = ["DpProcess", "DpHorizonProcess", "Repeated", "Composed", "CachedProcess", "EpsDelta", "Identity", "NonPrivate",
           "repeat", "compose", "cached", "eps_delta", "identity", "nonprivate", "clear_pld_cache"]
