"""``torchopt.transform`` stand-in: the elementary transformations the reference composes."""
from __future__ import annotations

from typing import Any, Callable, NamedTuple

import optree
import torch

from .base import EmptyState, GradientTransformation, identity


def _map(fn: Callable, *trees: Any) -> Any:
    return optree.tree_map(fn, *trees)


def scale(step_size: float) -> GradientTransformation:
    def update_fn(updates, state, *, params=None, inplace=True):
        if inplace:
            f = lambda g: g.mul_(step_size) if g is not None else None  # noqa: E731
        else:
            f = lambda g: g.mul(step_size) if g is not None else None  # noqa: E731
        return _map(f, updates), state

    return GradientTransformation(lambda params: EmptyState(), update_fn)


class ScaleByScheduleState(NamedTuple):
    count: Any


def scale_by_schedule(step_size_fn: Callable) -> GradientTransformation:
    def init_fn(params):
        leaves = [p for p in optree.tree_leaves(params) if isinstance(p, torch.Tensor)]
        dev = leaves[0].device if leaves else None
        return ScaleByScheduleState(count=torch.zeros(1, dtype=torch.int64, device=dev).squeeze_())

    def update_fn(updates, state, *, params=None, inplace=True):
        step_size = step_size_fn(state.count)
        if inplace:
            f = lambda g: g.mul_(step_size) if g is not None else None  # noqa: E731
        else:
            f = lambda g: g.mul(step_size) if g is not None else None  # noqa: E731
        return _map(f, updates), ScaleByScheduleState(count=state.count + 1)

    return GradientTransformation(init_fn, update_fn)


class AddDecayedWeightsState(NamedTuple):
    """No state."""


def add_decayed_weights(weight_decay: float = 0.0, mask: Any = None) -> GradientTransformation:
    if not weight_decay >= 0.0:
        raise ValueError(f"Invalid weight_decay value: {weight_decay}")
    if weight_decay == 0.0 and mask is None:
        return identity()
    if mask is not None:
        raise NotImplementedError("masked weight decay is not part of this stand-in")

    def update_fn(updates, state, *, params=None, inplace=True):
        assert params is not None, "Parameters are required for weight decay. Call `update(updates, state, params=params)`."
        if inplace:
            f = lambda g, p: g.add_(p.data, alpha=weight_decay) if g is not None else None  # noqa: E731
        else:
            f = lambda g, p: g.add(p, alpha=weight_decay) if g is not None else None  # noqa: E731
        return _map(f, updates, params), state

    return GradientTransformation(lambda params: AddDecayedWeightsState(), update_fn)


class TraceState(NamedTuple):
    trace: Any


def trace(momentum: float = 0.9, dampening: float = 0.0, nesterov: bool = False, moment_requires_grad: bool = False) -> GradientTransformation:
    if momentum == 0.0:
        return identity()

    def init_fn(params):
        return TraceState(trace=_map(lambda p: torch.zeros_like(p, requires_grad=moment_requires_grad), params))

    def update_fn(updates, state, *, params=None, inplace=True):
        if inplace:
            new_trace = _map(lambda g, t: t.mul_(momentum).add_(g, alpha=1.0 - dampening), updates, state.trace)
            if nesterov:
                updates = _map(lambda g, t: g.add_(t, alpha=momentum), updates, new_trace)
            else:
                updates = _map(lambda g, t: g.copy_(t), updates, new_trace)
        else:
            new_trace = _map(lambda g, t: t.mul(momentum).add(g, alpha=1.0 - dampening), updates, state.trace)
            updates = _map(lambda g, t: g.add(t, alpha=momentum), updates, new_trace) if nesterov else _map(lambda t: t.clone(), new_trace)
        return updates, TraceState(trace=new_trace)

    return GradientTransformation(init_fn, update_fn)


class ScaleByAdamState(NamedTuple):
    mu: Any
    nu: Any
    count: Any


def scale_by_adam(b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, eps_root: float = 0.0) -> GradientTransformation:
    def init_fn(params):
        z = lambda p: torch.zeros_like(p)  # noqa: E731
        return ScaleByAdamState(mu=_map(z, params), nu=_map(z, params), count=_map(lambda p: torch.zeros(1, dtype=torch.int64, device=p.device).squeeze_(), params))

    def update_fn(updates, state, *, params=None, inplace=True):
        mu = _map(lambda g, m: m.mul(b1).add(g, alpha=1 - b1), updates, state.mu)
        nu = _map(lambda g, v: v.mul(b2).addcmul(g, g, value=1 - b2), updates, state.nu)
        count = _map(lambda c: c + 1, state.count)
        out = _map(lambda m, v, c: (m / (1 - b1 ** c)) / ((v / (1 - b2 ** c) + eps_root).sqrt() + eps), mu, nu, count)
        return out, ScaleByAdamState(mu=mu, nu=nu, count=count)

    return GradientTransformation(init_fn, update_fn)
