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


@dataclass(frozen=True)
class ChainState:
    moment: Any
    count: int = 0


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

    def init(params):
        return ChainState(moment_scaler.init(params), 0)

    def update(updates, state: ChainState, *, params=None, inplace: bool = False):
        g, extra = route(updates)
        if weight_decay and not decoupled_weight_decay:
            if params is None:
                raise ConfigurationError("weight decay needs `params`")
            g = tree_map(lambda u, p: u + weight_decay * p.to(u.dtype), g, params)
        d, mom = moment_scaler.update(g, state.moment, params=params, **extra)
        if update_rms_clip is not None:
            d = clip_by_global_rms(d, float(update_rms_clip))
        if weight_decay and decoupled_weight_decay:
            if params is None:
                raise ConfigurationError("weight decay needs `params`")
            d = tree_map(lambda u, p: u + weight_decay * p.to(u.dtype), d, params)
        step = -resolve_lr(lr, state.count)
        return tree_map(lambda u: u * step, d), ChainState(mom, state.count + 1)

    return GradientTransformation(init, update)


__all__ = ["GradientTransformation", "ChainState", "apply_updates", "make_optimizer_chain", "clip_by_global_rms",
           "resolve_lr"]
