"""Privacy budgets: a target value for one metric of a process, used by ``calibrate`` and ``Accountant``.

Five kinds as in packages/opake-accounting/src/opake/api/accounting/core/_budgets.py:85-250: epsilon (at delta), delta
(at epsilon), advantage, beta (at alpha), Bayes risk (at prior). ``decreasing`` is True for privacy-loss metrics (safe
at or below the target) and False for privacy-gain metrics. Budgets serialize as ``{"type": name, **fields}``.
"""
from __future__ import annotations

from collections.abc import Callable, Mapping
from dataclasses import dataclass, fields
from threading import RLock
from typing import Any, Protocol, runtime_checkable

from ..base.exceptions import CheckpointError, PrivacyBudgetError


@runtime_checkable
class Budget(Protocol):
    @property
    def value(self) -> float: ...

    @property
    def name(self) -> str: ...

    @property
    def decreasing(self) -> bool: ...

    def evaluate(self, process) -> float: ...


def _unit(v, what):
    if not (0 < v < 1):
        raise PrivacyBudgetError(f"{what} must be in (0, 1), got {v}")


@dataclass(frozen=True)
class EpsilonBudget:
    epsilon: float
    delta: float

    def __post_init__(self):
        if self.epsilon <= 0:
            raise PrivacyBudgetError(f"epsilon must be > 0, got {self.epsilon}")
        _unit(self.delta, "delta")

    value = property(lambda s: s.epsilon)
    name = property(lambda s: f"epsilon({s.epsilon}, delta={s.delta})")
    decreasing = property(lambda s: True)

    def evaluate(self, process) -> float:
        return process.epsilon_at(self.delta)


@dataclass(frozen=True)
class DeltaBudget:
    delta: float
    epsilon: float

    def __post_init__(self):
        _unit(self.delta, "delta")
        if self.epsilon <= 0:
            raise PrivacyBudgetError(f"epsilon must be > 0, got {self.epsilon}")

    value = property(lambda s: s.delta)
    name = property(lambda s: f"delta({s.delta}, epsilon={s.epsilon})")
    decreasing = property(lambda s: True)

    def evaluate(self, process) -> float:
        return process.delta_at(self.epsilon)


@dataclass(frozen=True)
class AdvantageBudget:
    advantage: float

    def __post_init__(self):
        _unit(self.advantage, "advantage")

    value = property(lambda s: s.advantage)
    name = property(lambda s: f"advantage({s.advantage})")
    decreasing = property(lambda s: True)

    def evaluate(self, process) -> float:
        return process.advantage()


@dataclass(frozen=True)
class BetaBudget:
    beta: float
    alpha: float

    def __post_init__(self):
        _unit(self.beta, "beta")
        _unit(self.alpha, "alpha")

    value = property(lambda s: s.beta)
    name = property(lambda s: f"beta({s.beta}, alpha={s.alpha})")
    decreasing = property(lambda s: False)

    def evaluate(self, process) -> float:
        return process.beta_at(self.alpha)


@dataclass(frozen=True)
class RiskBudget:
    risk: float
    prior: float

    def __post_init__(self):
        _unit(self.risk, "risk")
        _unit(self.prior, "prior")

    value = property(lambda s: s.risk)
    name = property(lambda s: f"risk({s.risk}, prior={s.prior})")
    decreasing = property(lambda s: False)

    def evaluate(self, process) -> float:
        return process.risk_at(self.prior)


_LOCK = RLock()
_SAVE: dict[type, tuple[str, Callable]] = {}
_LOAD: dict[str, Callable] = {}
_TYPES: dict[str, type] = {}


def register_budget_serializer(typ: type, state_dict_fn, from_state_dict_fn, *, type_name: str | None = None) -> None:
    with _LOCK:
        name = type_name or f"{typ.__module__}.{typ.__qualname__}"
        if _TYPES.get(name, typ) is not typ:
            raise CheckpointError(f"Budget checkpoint type name already registered: {name}")
        old = _SAVE.get(typ)
        if old is not None and old[0] != name:
            _LOAD.pop(old[0], None)
            _TYPES.pop(old[0], None)
        _SAVE[typ], _LOAD[name], _TYPES[name] = (name, state_dict_fn), from_state_dict_fn, typ


def budget_state_dict(budget) -> dict[str, Any]:
    with _LOCK:
        entry = _SAVE.get(type(budget))
    if entry is None:
        raise CheckpointError(f"Cannot serialize budget {type(budget).__qualname__}: no budget serializer is registered. "
                              "Register one with `register_budget_serializer`.")
    state = dict(entry[1](budget))
    if "type" in state:
        raise CheckpointError("Budget serializer returned reserved key 'type'.")
    return {"type": entry[0]} | state


def budget_from_state_dict(state: Mapping[str, Any]):
    data = dict(state)
    if "type" not in data:
        raise CheckpointError("Budget checkpoint is missing required key 'type'.")
    name = data.pop("type")
    with _LOCK:
        fn = _LOAD.get(name)
    if fn is None:
        raise CheckpointError(f"Cannot restore budget type {name!r}: no budget serializer is registered.")
    return fn(data)


for _cls in (EpsilonBudget, DeltaBudget, AdvantageBudget, BetaBudget, RiskBudget):
    register_budget_serializer(_cls, lambda b: {f.name: getattr(b, f.name) for f in fields(b)},
                               lambda st, c=_cls: c(**dict(st)), type_name=_cls.__name__)


def epsilon_budget(epsilon: float, delta: float) -> EpsilonBudget:
    return EpsilonBudget(epsilon, delta)


def delta_budget(delta: float, epsilon: float) -> DeltaBudget:
    return DeltaBudget(delta, epsilon)


def advantage_budget(advantage: float) -> AdvantageBudget:
    return AdvantageBudget(advantage)


def beta_budget(beta: float, alpha: float) -> BetaBudget:
    return BetaBudget(beta, alpha)


def risk_budget(risk: float, prior: float = 0.5) -> RiskBudget:
    return RiskBudget(risk, prior)


__all__ = ["Budget", "EpsilonBudget", "DeltaBudget", "AdvantageBudget", "BetaBudget", "RiskBudget", "epsilon_budget",
           "delta_budget", "advantage_budget", "beta_budget", "risk_budget", "register_budget_serializer",
           "budget_state_dict", "budget_from_state_dict"]
