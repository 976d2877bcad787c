"""Learning-rate schedule factory: Hugging Face scheduler names (or a schedule recipe) to a ``step -> lr`` callable
built from ``engine.scheduling`` (packages/opake-transformers/src/opake/api/transformers/trainer/_scheduler.py:70-383).

Every name accepts exactly the keyword arguments Hugging Face documents for it; anything else is a configuration
error, as is a schedule recipe combined with ``warmup_steps`` / ``lr_scheduler_kwargs`` (compose the warm-up into the
recipe instead). ``warmup_steps`` below 1 is a fraction of the run."""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Callable

from ..base.exceptions import ConfigurationError
from ..engine import scheduling as S

__all__ = ["build_lr_schedule", "get_warmup_steps", "SUPPORTED_SCHEDULERS"]

_WSD = frozenset({"num_decay_steps", "num_stable_steps", "warmup_type", "decay_type", "min_lr_ratio", "num_cycles"})
SUPPORTED_SCHEDULERS: dict[str, frozenset] = {
    "constant": frozenset(),
    "constant_with_warmup": frozenset(),
    "linear": frozenset(),
    "cosine": frozenset({"num_cycles"}),
    "polynomial": frozenset({"lr_end", "power"}),
    "inverse_sqrt": frozenset({"timescale"}),
    "cosine_with_restarts": frozenset({"num_cycles"}),
    "cosine_with_min_lr": frozenset({"num_cycles", "min_lr", "min_lr_rate"}),
    "cosine_warmup_with_min_lr": frozenset({"num_cycles", "min_lr", "min_lr_rate", "warmup_lr_rate"}),
    "warmup_stable_decay": _WSD,
    # shapes of ``engine.scheduling`` without a Hugging Face name of their own
    "exponential": frozenset({"decay_rate", "transition_steps"}),
    "one_minus_sqrt": frozenset(),
}
_WSD_SHAPES = ("linear", "cosine", "1-sqrt")


def get_warmup_steps(num_training_steps: int, warmup_steps: int | float) -> int:
    """``>= 1``: a step count (truncated); in ``(0, 1)``: that fraction of the run, rounded up."""
    if warmup_steps >= 1:
        return int(warmup_steps)
    return math.ceil(num_training_steps * warmup_steps)


@dataclasses.dataclass(frozen=True)
class _CosineSpan:
    """``end + (init - end) * (1 + cos(2 pi cycles f)) / 2`` over ``steps`` (held at its last value afterwards)."""

    init_value: float
    end_value: float
    steps: float
    num_cycles: float = 0.5

    def __call__(self, step: int) -> float:
        f = 1.0 if self.steps <= 0 else min(max(step / self.steps, 0.0), 1.0)
        c = 0.5 * (1.0 + math.cos(2.0 * math.pi * self.num_cycles * f))
        return self.end_value + (self.init_value - self.end_value) * max(0.0, c)


@dataclasses.dataclass(frozen=True)
class _CosineRestarts:
    """Hard restarts with a REAL-valued cycle length ``steps / cycles``: the k-th restart sits at ``k * steps / cycles``
    even when that is not an integer, which is what the fractional-progress formula of Hugging Face gives."""

    init_value: float
    steps: int
    cycles: int

    def __call__(self, step: int) -> float:
        if step >= self.steps:
            return 0.0
        f = max(step, 0) / max(self.steps, 1)
        return self.init_value * 0.5 * (1.0 + math.cos(math.pi * ((self.cycles * f) % 1.0)))


@dataclasses.dataclass(frozen=True)
class _HoldAfter:
    schedule: Callable[[int], float]
    end: int
    floor: float

    def __call__(self, step: int) -> float:
        return self.floor if step >= self.end else self.schedule(step)


def _min_lr(base_lr: float, kw: dict) -> float:
    a, r = kw.get("min_lr"), kw.get("min_lr_rate")
    if a is not None and r is not None:
        raise ConfigurationError("set only one of min_lr or min_lr_rate")
    if a is not None:
        return float(a)
    if r is not None:
        return float(r) * base_lr
    raise ConfigurationError("lr_scheduler_kwargs must include exactly one of {'min_lr': ...} or {'min_lr_rate': ...}")


def _wsd(base_lr: float, W: int, total: int, kw: dict) -> Callable[[int], float]:
    warmup_type, decay_type = kw.get("warmup_type", "linear"), kw.get("decay_type", "cosine")
    if warmup_type not in _WSD_SHAPES:
        raise ConfigurationError(f"warmup_stable_decay warmup_type must be one of {sorted(_WSD_SHAPES)}; got {warmup_type!r}")
    if decay_type not in _WSD_SHAPES:
        raise ConfigurationError(f"warmup_stable_decay decay_type must be one of {sorted(_WSD_SHAPES)}; got {decay_type!r}")
    if "num_decay_steps" not in kw:
        raise ConfigurationError("warmup_stable_decay requires lr_scheduler_kwargs={'num_decay_steps': ...}")
    D = int(kw["num_decay_steps"])
    stable = int(kw.get("num_stable_steps", total - W - D))
    floor = float(kw.get("min_lr_ratio", 0.0)) * base_lr
    if decay_type == "cosine":      # the cosine keeps oscillating past its span, so the tail is pinned to the floor
        tail = _HoldAfter(_CosineSpan(base_lr, floor, D, float(kw.get("num_cycles", 0.5))), D, floor)
    elif decay_type == "linear":
        tail = S.linear_schedule(base_lr, floor, D)
    else:
        tail = S.one_minus_sqrt_schedule(base_lr, D, end_value=floor)

    def after_warmup(step: int) -> float:
        return base_lr if step < stable else tail(step - stable)

    if W <= 0:
        return after_warmup
    return S.with_warmup(after_warmup, W, init_value=floor, warmup_type=warmup_type)      # ramp: floor -> base_lr


def build_lr_schedule(name_or_args: Any, num_training_steps: int | None = None, *, learning_rate: float | None = None,
                      total_steps: int | None = None, warmup_steps: int | float = 0, kwargs: dict | None = None
                      ) -> Callable[[int], float]:
    """``build_lr_schedule(args, num_training_steps)`` reads ``lr_scheduler``, ``warmup_steps``, ``learning_rate`` and
    ``lr_scheduler_kwargs`` from a training-arguments object; ``build_lr_schedule(name, learning_rate=..., total_steps=...,
    warmup_steps=..., kwargs=...)`` is the explicit form. ``total_steps`` counts the warm-up."""
    if not isinstance(name_or_args, str) and not callable(name_or_args) and hasattr(name_or_args, "lr_scheduler"):
        a = name_or_args
        return build_lr_schedule(a.lr_scheduler, learning_rate=a.learning_rate, total_steps=num_training_steps,
                                 warmup_steps=a.warmup_steps or 0, kwargs=a.lr_scheduler_kwargs)
    name = getattr(name_or_args, "value", name_or_args)
    if not isinstance(name, str) and callable(name):        # a schedule recipe: returned as it is
        if warmup_steps:
            raise ConfigurationError("warmup_steps is incompatible with a user-supplied lr_scheduler schedule; compose "
                                     "with_warmup(schedule, ...) into the recipe")
        if kwargs:
            raise ConfigurationError("lr_scheduler_kwargs is incompatible with a user-supplied lr_scheduler schedule; "
                                     "configure the recipe through its constructor")
        return name
    total = int(total_steps if total_steps is not None else num_training_steps)
    kw = dict(kwargs or {})
    if name not in SUPPORTED_SCHEDULERS:
        raise ConfigurationError(f"unknown lr_scheduler {name!r}; supported: {sorted(SUPPORTED_SCHEDULERS)}")
    extra = set(kw) - SUPPORTED_SCHEDULERS[name]
    if extra:
        raise ConfigurationError(f"lr_scheduler_kwargs contains unsupported keys for lr_scheduler={name!r}: {sorted(extra)}; "
                                 f"allowed: {sorted(SUPPORTED_SCHEDULERS[name]) or '<none>'}")
    lr = float(learning_rate)
    W = get_warmup_steps(total, warmup_steps)
    decay_steps = max(1, total - W)
    warmup_init = 0.0
    if name == "constant":
        return S.constant_schedule(lr)
    if name == "warmup_stable_decay":
        return _wsd(lr, W, total, kw)
    if name == "constant_with_warmup":
        decay = S.constant_schedule(lr)
    elif name == "linear":
        decay = S.linear_schedule(lr, 0.0, decay_steps)
    elif name == "cosine":
        decay = _CosineSpan(lr, 0.0, decay_steps, float(kw.get("num_cycles", 0.5)))
    elif name == "polynomial":
        lr_end = float(kw.get("lr_end", 1e-7))
        if lr_end >= lr:
            raise ConfigurationError(f"lr_end ({lr_end}) must be smaller than initial lr ({lr})")
        decay = S.polynomial_schedule(lr, lr_end, float(kw.get("power", 1.0)), decay_steps)
    elif name == "inverse_sqrt":
        ts = kw.get("timescale")            # an explicit 0 is the caller's error, not a request for the default
        ts = ts if ts is not None else (W or 10_000)
        if ts <= 0:
            raise ConfigurationError(f"inverse_sqrt timescale must be positive; got {ts}")
        decay = S.inverse_sqrt_schedule(lr, timescale=int(ts))
    elif name == "cosine_with_restarts":
        decay = _CosineRestarts(lr, decay_steps, int(kw.get("num_cycles", 1)))
    elif name in ("cosine_with_min_lr", "cosine_warmup_with_min_lr"):
        decay = _CosineSpan(lr, _min_lr(lr, kw), decay_steps, float(kw.get("num_cycles", 0.5)))
        if name == "cosine_warmup_with_min_lr":
            # ramp r + (1 - r) * step / W (upstream anchors the same ramp at W - 1: equal at both ends, not inside)
            warmup_init = float(kw.get("warmup_lr_rate") or 0.0) * lr
    elif name == "exponential":
        decay = S.exponential_schedule(lr, float(kw.get("decay_rate", 0.5)), int(kw.get("transition_steps", decay_steps)))
    else:       # one_minus_sqrt
        decay = S.one_minus_sqrt_schedule(lr, decay_steps)
    return S.with_warmup(decay, W, init_value=warmup_init) if W > 0 else decay
