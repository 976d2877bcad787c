"""Learning-rate schedule factory: Hugging Face scheduler names to the schedule callables of ``engine.scheduling``
(packages/opake-transformers/src/opake/api/transformers/trainer/_scheduler.py:70-383)."""
from __future__ import annotations

from typing import Callable

from ..base.exceptions import ConfigurationError
from ..engine import scheduling as S

__all__ = ["build_lr_schedule"]


def build_lr_schedule(name: str, *, learning_rate: float, total_steps: int, warmup_steps: int = 0,
                      kwargs: dict | None = None) -> Callable[[int], float]:
    """Returns ``step -> lr``. ``warmup_steps`` of linear warm-up precede every decay shape; ``total_steps`` counts
    the warm-up."""
    kw = dict(kwargs or {})
    decay_steps = max(1, total_steps - warmup_steps)
    lr = float(learning_rate)

    def warm(schedule):
        return S.with_warmup(schedule, warmup_steps, init_value=0.0) if warmup_steps > 0 else schedule

    if name == "linear":
        return warm(S.linear_schedule(lr, float(kw.get("end_value", 0.0)), decay_steps))
    if name == "cosine":
        return warm(S.cosine_schedule(lr, decay_steps, alpha=float(kw.get("min_lr_rate", kw.get("alpha", 0.0))),
                                      num_cycles=float(kw.get("num_cycles", 0.5))))
    if name == "cosine_with_restarts":
        cycles = int(kw.get("num_cycles", 1))
        return warm(S.with_restarts(S.cosine_schedule(lr, max(1, decay_steps // max(1, cycles))),
                                    max(1, decay_steps // max(1, cycles))))
    if name == "polynomial":
        return warm(S.polynomial_schedule(lr, float(kw.get("lr_end", 1e-7)), float(kw.get("power", 1.0)), decay_steps))
    if name == "constant":
        return S.constant_schedule(lr)
    if name == "constant_with_warmup":
        return warm(S.constant_schedule(lr))
    if name == "inverse_sqrt":
        return warm(S.inverse_sqrt_schedule(lr, timescale=int(kw.get("timescale", max(1, warmup_steps)))))
    if name == "exponential":
        return warm(S.exponential_schedule(lr, float(kw.get("decay_rate", 0.5)), int(kw.get("transition_steps", decay_steps))))
    if name == "one_minus_sqrt":
        return warm(S.one_minus_sqrt_schedule(lr, decay_steps))
    if name == "warmup_stable_decay":
        n_decay = int(kw.get("num_decay_steps", max(1, int(0.1 * total_steps))))
        n_stable = int(kw.get("num_stable_steps", max(0, total_steps - warmup_steps - n_decay)))
        return S.warmup_stable_decay(lr, warmup_steps, n_stable, n_decay, end_value=lr * float(kw.get("min_lr_ratio", 0.0)),
                                     warmup_type=kw.get("warmup_type", "linear"), decay_type=kw.get("decay_type", "linear"))
    raise ConfigurationError(f"unknown lr_scheduler {name!r}")
