"""Bisection calibration of one scalar parameter (noise multiplier, sample rate, steps) against a privacy budget.

Contract of packages/opake-accounting/src/opake/api/accounting/core/calibration.py:70-552: the metric must be monotone
in the parameter on ``[param_min, param_max]``; which endpoint is privacy-safe is found by probing both; the result is
one-sided (never under-noised): loss metrics end at or below the target, gain metrics at or above, within the relative
``tolerance`` (default 1e-6) or the call raises :class:`CalibrationError`.
"""
from __future__ import annotations

import math
from collections.abc import Callable
from dataclasses import dataclass

from ..base.exceptions import CalibrationError
from .budgets import Budget, epsilon_budget, delta_budget, advantage_budget, beta_budget, risk_budget  # noqa: F401
from .core import DpProcess


@dataclass(frozen=True)
class CalibrateResult:
    param: float
    achieved: float
    target: float
    iterations: int
    converged: bool
    mc_failure_probability: float = 0.0

    @property
    def mc_confidence(self) -> float:
        return 1.0 - self.mc_failure_probability

    def __repr__(self) -> str:
        status = "converged" if self.converged else "max iterations"
        return (f"CalibrateResult(param={self.param:.6f}, achieved={self.achieved:.6f}, target={self.target:.6f}, "
                f"iterations={self.iterations}, {status})")


def calibrate(budget: Budget, process: Callable[[float], DpProcess], param_min: float, param_max: float,
              tolerance: float = 1e-6, max_iterations: int = 100, prefix: DpProcess | None = None) -> CalibrateResult:
    if not (math.isfinite(param_min) and math.isfinite(param_max)) or not param_min < param_max:
        raise CalibrationError(f"need finite param_min < param_max, got [{param_min}, {param_max}]")
    if not (tolerance > 0 and math.isfinite(tolerance)):
        raise CalibrationError(f"tolerance must be positive and finite, got {tolerance}")
    if max_iterations < 1:
        raise CalibrationError(f"max_iterations must be >= 1, got {max_iterations}")
    target = float(budget.value)

    def metric(x: float) -> float:
        p = process(x)
        if prefix is not None:
            p = prefix | p
        return float(budget.evaluate(p))

    def safe(v: float) -> bool:
        return v <= target if budget.decreasing else v >= target

    lo, hi = float(param_min), float(param_max)
    v_lo, v_hi = metric(lo), metric(hi)
    if safe(v_lo) == safe(v_hi):
        side = "both endpoints already satisfy" if safe(v_lo) else "neither endpoint satisfies"
        if safe(v_lo):
            # a whole-interval-safe search still has a best (least noisy / most useful) end: the one closer to target
            best = (lo, v_lo) if abs(v_lo - target) <= abs(v_hi - target) else (hi, v_hi)
            if math.isclose(best[1], target, rel_tol=tolerance, abs_tol=0.0):
                return CalibrateResult(best[0], best[1], target, 0, True)
        raise CalibrationError(f"cannot bracket target {budget.name}: {side} it (metric {v_lo:.6g} at {lo}, {v_hi:.6g} at "
                               f"{hi}); widen or move the search interval")
    if v_lo == v_hi:
        raise CalibrationError("metric is flat over the search interval")
    # orient: s = safe end, u = unsafe end
    s, v_s, u = (lo, v_lo, hi) if safe(v_lo) else (hi, v_hi, lo)
    it = 0
    for it in range(1, max_iterations + 1):
        if math.isclose(v_s, target, rel_tol=tolerance, abs_tol=0.0):
            return CalibrateResult(s, v_s, target, it - 1, True)
        mid = 0.5 * (s + u)
        if mid == s or mid == u:
            break
        v_mid = metric(mid)
        if safe(v_mid):
            s, v_s = mid, v_mid
        else:
            u = mid
    if math.isclose(v_s, target, rel_tol=max(tolerance, 1e-3), abs_tol=0.0) or abs(s - u) <= 1e-12 * max(1.0, abs(s)):
        return CalibrateResult(s, v_s, target, it, math.isclose(v_s, target, rel_tol=tolerance, abs_tol=0.0))
    raise CalibrationError(f"calibration did not reach {budget.name} within {max_iterations} iterations "
                           f"(best safe parameter {s} achieves {v_s})")


__all__ = ["CalibrateResult", "calibrate", "epsilon_budget", "delta_budget", "advantage_budget", "beta_budget",
           "risk_budget"]
