"""Immutable running privacy ledger: ``acct = acct | step``; metrics are evaluated lazily on the composed process
(packages/opake-accounting/src/opake/api/accounting/core/_accountant.py:39-263)."""
from __future__ import annotations

from typing import Any

from ..base.exceptions import CheckpointError
from ..base.serialization import register_serializer
from .budgets import Budget, budget_from_state_dict, budget_state_dict
from .codec import process_from_dict, process_to_dict
from .core import DpProcess, Identity


class Accountant:
    def __init__(self, budget: Budget | None = None, prefix: DpProcess | None = None) -> None:
        self.process: DpProcess = Identity() if prefix is None else prefix
        self._budget = budget

    def __or__(self, process: DpProcess) -> "Accountant":
        return Accountant(self._budget, self.process | process)

    def epsilon_at(self, delta: float) -> float:
        return self.process.epsilon_at(delta)

    def delta_at(self, epsilon: float) -> float:
        return self.process.delta_at(epsilon)

    def advantage(self) -> float:
        return self.process.advantage()

    def beta_at(self, alpha: float) -> float:
        return self.process.beta_at(alpha)

    def risk_at(self, prior: float) -> float:
        return self.process.risk_at(prior)

    @property
    def budget(self):
        return self._budget

    @property
    def budget_exceeded(self) -> bool:
        if self._budget is None:
            return False
        got = self._budget.evaluate(self.process)
        return got > self._budget.value if self._budget.decreasing else got < self._budget.value

    def state_dict(self) -> dict[str, Any]:
        return _save(self)

    def __repr__(self) -> str:
        return f"Accountant(process={self.process!r}, budget={self._budget!r})"


def _save(a: Accountant) -> dict[str, Any]:
    out: dict[str, Any] = {"process": process_to_dict(a.process)}
    if a._budget is not None:
        out["budget"] = budget_state_dict(a._budget)
    return out


def _load(template: Accountant, state) -> Accountant:
    state = dict(state)
    budget = template._budget
    saved = state.get("budget")
    if saved is not None:
        budget = budget_from_state_dict(dict(saved))
        if template._budget is not None and budget_state_dict(budget) != budget_state_dict(template._budget):
            raise CheckpointError(f"Accountant checkpoint budget {budget.name!r} (value={budget.value!r}) does not match "
                                  f"template budget {template._budget.name!r} (value={template._budget.value!r}). Restore "
                                  "with Accountant() to use the checkpoint budget. To replace it, construct a new "
                                  "Accountant with the restored process as prefix.")
    return Accountant(budget, process_from_dict(dict(state["process"])))


register_serializer(Accountant, _save, _load)

__all__ = ["Accountant"]
