"""Learning-rate (and general scalar) schedules as frozen callable dataclasses ``step -> value``.

Same catalogue as packages/opake-engine/src/opake/api/engine/scheduling/__init__.py:22-44: constant, cosine,
exponential, inverse-sqrt, linear, one-minus-sqrt, polynomial, warmup-stable-decay, restarts and warmup wrappers,
plus the named ramp/decay shape tables used by the trainer.
"""
from __future__ import annotations

import math
from collections.abc import Callable
from dataclasses import dataclass

from ..base.exceptions import ConfigurationError

Schedule = Callable[[int], float]


def _frac(step: int, total: int) -> float:
    return 1.0 if total <= 0 else min(max(step / total, 0.0), 1.0)


@dataclass(frozen=True)
class constant_schedule:
    value: float

    def __call__(self, step: int) -> float:
        return float(self.value)


@dataclass(frozen=True)
class linear_schedule:
    init_value: float
    end_value: float
    transition_steps: int
    transition_begin: int = 0

    def __call__(self, step: int) -> float:
        f = _frac(step - self.transition_begin, self.transition_steps)
        return self.init_value + (self.end_value - self.init_value) * f


@dataclass(frozen=True)
class cosine_schedule:
    init_value: float
    decay_steps: int
    alpha: float = 0.0
    num_cycles: float = 0.5

    def __call__(self, step: int) -> float:
        f = _frac(step, self.decay_steps)
        cos = 0.5 * (1.0 + math.cos(math.pi * 2.0 * self.num_cycles * f))
        return self.init_value * ((1.0 - self.alpha) * max(0.0, cos) + self.alpha)


@dataclass(frozen=True)
class exponential_schedule:
    init_value: float
    decay_rate: float
    transition_steps: int = 1
    staircase: bool = False
    end_value: float | None = None

    def __call__(self, step: int) -> float:
        p = step / max(self.transition_steps, 1)
        if self.staircase:
            p = math.floor(p)
        v = self.init_value * self.decay_rate**p
        if self.end_value is not None:
            v = max(v, self.end_value) if self.decay_rate < 1 else min(v, self.end_value)
        return v


@dataclass(frozen=True)
class inverse_sqrt_schedule:
    init_value: float
    timescale: int = 1

    def __call__(self, step: int) -> float:
        return self.init_value / math.sqrt(max(step, 0) / max(self.timescale, 1) + 1.0)


@dataclass(frozen=True)
class one_minus_sqrt_schedule:
    init_value: float
    decay_steps: int
    end_value: float = 0.0

    def __call__(self, step: int) -> float:
        f = _frac(step, self.decay_steps)
        return self.end_value + (self.init_value - self.end_value) * (1.0 - math.sqrt(f))


@dataclass(frozen=True)
class polynomial_schedule:
    init_value: float
    end_value: float
    power: float
    transition_steps: int
    transition_begin: int = 0

    def __call__(self, step: int) -> float:
        f = _frac(step - self.transition_begin, self.transition_steps)
        return (self.init_value - self.end_value) * (1.0 - f) ** self.power + self.end_value


def _ramp_linear(f: float) -> float:
    return f


def _ramp_cosine(f: float) -> float:
    return 0.5 * (1.0 - math.cos(math.pi * f))


def _ramp_sqrt(f: float) -> float:
    return math.sqrt(f)


NAMED_RAMPS = {"linear": _ramp_linear, "cosine": _ramp_cosine, "1-sqrt": lambda f: 1.0 - math.sqrt(1.0 - f), "sqrt": _ramp_sqrt}
NAMED_DECAYS = {"linear": lambda f: 1.0 - f, "cosine": lambda f: 0.5 * (1.0 + math.cos(math.pi * f)),
                "1-sqrt": lambda f: 1.0 - math.sqrt(f)}


@dataclass(frozen=True)
class warmup_stable_decay:
    peak_value: float
    warmup_steps: int
    stable_steps: int
    decay_steps: int
    init_value: float = 0.0
    end_value: float = 0.0
    warmup_type: str = "linear"
    decay_type: str = "linear"

    def __post_init__(self):
        if self.warmup_type not in NAMED_RAMPS or self.decay_type not in NAMED_DECAYS:
            raise ConfigurationError(f"unknown ramp/decay type {self.warmup_type!r}/{self.decay_type!r}")

    def __call__(self, step: int) -> float:
        if step < self.warmup_steps:
            r = NAMED_RAMPS[self.warmup_type](_frac(step, self.warmup_steps))
            return self.init_value + (self.peak_value - self.init_value) * r
        s = step - self.warmup_steps
        if s < self.stable_steps:
            return self.peak_value
        d = NAMED_DECAYS[self.decay_type](_frac(s - self.stable_steps, self.decay_steps))
        return self.end_value + (self.peak_value - self.end_value) * d


@dataclass(frozen=True)
class with_warmup:
    schedule: Schedule
    warmup_steps: int
    init_value: float = 0.0
    warmup_type: str = "linear"

    def __call__(self, step: int) -> float:
        if step < self.warmup_steps:
            target = self.schedule(0)
            return self.init_value + (target - self.init_value) * NAMED_RAMPS[self.warmup_type](_frac(step, self.warmup_steps))
        return self.schedule(step - self.warmup_steps)


@dataclass(frozen=True)
class with_restarts:
    schedule: Schedule
    period: int
    decay: float = 1.0

    def __call__(self, step: int) -> float:
        cycle, pos = divmod(max(step, 0), max(self.period, 1))
        return self.schedule(pos) * self.decay**cycle


__all__ = ["constant_schedule", "cosine_schedule", "exponential_schedule", "inverse_sqrt_schedule", "linear_schedule",
           "one_minus_sqrt_schedule", "polynomial_schedule", "warmup_stable_decay", "with_restarts", "with_warmup",
           "NAMED_DECAYS", "NAMED_RAMPS"]
