"""Optimizer chain: moment scaling -> optional global-RMS clip -> weight decay -> ``-lr`` scaling.

Mirrors the routing rules of packages/opake-optimizers/src/opake/api/optimizers/_chain.py:86-284 without torchopt:
``update()`` accepts a ``NoisedPytree`` (its ``noise_stddev`` is forwarded to moment scalers that use it), a
``SecondMomentNoiseOutput`` (forwarded as ``noisy_squared_grads`` to scalers that accept it) or a raw pytree; a bare
``ClippedPytree`` is rejected because it has not been through a noise mechanism. Decoupled weight decay (AdamW) is
applied after moment scaling, L2 decay before it.
"""
from __future__ import annotations

import inspect
from collections.abc import Callable
from dataclasses import dataclass
from typing import Any, NamedTuple

import torch

from ..base.exceptions import ConfigurationError, InputTypeError
from ..engine.pytree import tree_leaves, tree_map
from ..engine.types import ClippedPytree, NoisedPytree, SecondMomentNoiseOutput

LR = Any  # float or schedule(step) -> float


class GradientTransformation(NamedTuple):
    init: Callable[[Any], Any]
    update: Callable[..., tuple[Any, Any]]


class ScaleByScheduleState(NamedTuple):
    """State of the ``-lr`` scaling when ``lr`` is a schedule: the number of updates so far."""

    count: torch.Tensor


class ChainState(tuple):
    """State of an optimizer chain: one entry per stage, in stage order, as the reference's chain keeps it
    (packages/opake-optimizers/src/opake/api/optimizers/_chain.py:224-284), so that serialized optimizer states have
    the same flat keys (``[0].mu.<leaf>``, ``[0].step``, ``[3].count``, ...). Decoupled decay (AdamW):
    ``(moment, rms clip, weight decay, lr)``; L2 decay: ``(weight decay, moment, rms clip, lr)``. Stages without state
    hold an empty tuple."""

    __slots__ = ()

    def __new__(cls, stages):
        return super().__new__(cls, stages)

    @property
    def moment(self):
        return self[_moment_index(self)]

    @property
    def count(self) -> int:
        lr_state = self[3]
        return int(lr_state.count) if isinstance(lr_state, ScaleByScheduleState) else 0


def _moment_index(state: tuple) -> int:
    # the moment stage is the first one that carries state other than the (stateless) decay / clip stages
    for i in (0, 1):
        if state[i] != ():
            return i
    return 0


def apply_updates(params: Any, updates: Any, *, inplace: bool = False) -> Any:
    if inplace:
        def add_(p, u):
            p.add_(u.to(p.dtype))
            return p

        return tree_map(add_, params, updates)
    return tree_map(lambda p, u: p + u.to(p.dtype), params, updates)


def resolve_lr(lr: LR, count: int) -> float:
    return float(lr(count)) if callable(lr) else float(lr)


def clip_by_global_rms(updates: Any, threshold: float) -> Any:
    leaves = tree_leaves(updates)
    if not leaves:
        return updates
    sq = sum(l.detach().double().pow(2).sum() for l in leaves)
    n = sum(l.numel() for l in leaves)
    scale = torch.clamp((sq / n).sqrt() / threshold, min=1.0)
    return tree_map(lambda u: u / scale.to(u.dtype), updates)


def _unsupported_second_moment(name: str):
    raise InputTypeError(f"{name} does not consume a private second-moment stream; pass `.noisy_grads` or use an "
                         "optimizer with a second-moment accumulator (adam, adamw, rmsprop, adagrad).")


def make_optimizer_chain(moment_scaler: GradientTransformation, lr: LR, weight_decay: float, *, optimizer_name: str,
                         decoupled_weight_decay: bool = True, update_rms_clip: float | None = None):
    if weight_decay < 0:
        raise ConfigurationError(f"weight_decay must be >= 0, got {weight_decay}")
    sig = inspect.signature(moment_scaler.update).parameters
    varkw = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.values())
    takes_std = "noise_stddev" in sig or varkw
    takes_sq = "noisy_squared_grads" in sig

    def route(updates):
        if isinstance(updates, SecondMomentNoiseOutput):
            if not takes_sq:
                _unsupported_second_moment(optimizer_name)
            g, s = updates.noisy_grads, updates.noisy_squared_grads
            for nm, v in (("noisy_grads", g), ("noisy_squared_grads", s)):
                if isinstance(v, ClippedPytree) and not isinstance(v, NoisedPytree):
                    raise InputTypeError(f"SecondMomentNoiseOutput.{nm} is a ClippedPytree that has not passed through a "
                                         "noise mechanism.")
            unwrap = (lambda v: v.pytree if isinstance(v, NoisedPytree) else v)
            return unwrap(g), {"noisy_squared_grads": unwrap(s)}
        if isinstance(updates, NoisedPytree):
            return updates.pytree, ({"noise_stddev": updates.noise_stddev} if takes_std else {})
        if isinstance(updates, ClippedPytree):
            raise InputTypeError("optimizer.update() received ClippedPytree updates that have not passed through a noise "
                                 "mechanism. Pass NoisedPytree outputs from a DP mechanism, or unwrap `.pytree` "
                                 "explicitly for non-private use.")
        return updates, {}

    scheduled = callable(lr)
    m_at = 0 if decoupled_weight_decay else 1

    def pack(mom, count):
        lr_state = ScaleByScheduleState(torch.tensor(int(count), dtype=torch.int64)) if scheduled else ()
        stages = [(), (), (), lr_state]
        stages[m_at] = mom
        return ChainState(stages)

    def init(params):
        return pack(moment_scaler.init(params), 0)

    def update(updates, state: ChainState, *, params=None, inplace: bool = False):
        g, extra = route(updates)
        if weight_decay and not decoupled_weight_decay:
            if params is None:
                raise ConfigurationError("weight decay needs `params`")
            g = tree_map(lambda u, p: u + weight_decay * p.to(u.dtype), g, params)
        count = int(state[3].count) if scheduled else 0
        d, mom = moment_scaler.update(g, state[m_at], params=params, **extra)
        if update_rms_clip is not None:
            d = clip_by_global_rms(d, float(update_rms_clip))
        if weight_decay and decoupled_weight_decay:
            if params is None:
                raise ConfigurationError("weight decay needs `params`")
            d = tree_map(lambda u, p: u + weight_decay * p.to(u.dtype), d, params)
        step = -resolve_lr(lr, count)
        return tree_map(lambda u: u * step, d), pack(mom, count + 1)

    return GradientTransformation(init, update)


__all__ = ["GradientTransformation", "ChainState", "ScaleByScheduleState", "apply_updates", "make_optimizer_chain", "clip_by_global_rms",
           "resolve_lr"]
