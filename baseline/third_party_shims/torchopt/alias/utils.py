"""``torchopt.alias.utils`` stand-in."""
from __future__ import annotations

from typing import Any, Callable

import optree

from ..base import EmptyState, GradientTransformation, identity
from ..transform import scale, scale_by_schedule


def scale_by_neg_lr(lr: float | Callable) -> GradientTransformation:
    """Multiply the updates by ``-lr``; ``lr`` may be a schedule called with the step count."""
    if callable(lr):
        return scale_by_schedule(lambda count: -lr(count))
    if not lr >= 0.0:
        raise ValueError(f"Invalid learning rate: {lr}")
    return scale(-lr)


def flip_sign_and_add_weight_decay(weight_decay: float = 0.0, maximize: bool = False) -> GradientTransformation:
    """Negate the gradient when maximising and add ``weight_decay * params`` (L2 form)."""
    if not weight_decay >= 0.0:
        raise ValueError(f"Invalid weight_decay value: {weight_decay}")
    if not maximize and weight_decay == 0.0:
        return identity()

    def update_fn(updates: Any, state: Any, *, params: Any = None, inplace: bool = True):
        if weight_decay != 0.0:
            assert params is not None, "Parameters are required for weight decay."
        if inplace:
            if maximize:
                updates = optree.tree_map(lambda g: g.neg_(), updates)
            if weight_decay != 0.0:
                updates = optree.tree_map(lambda g, p: g.add_(p.data, alpha=weight_decay), updates, params)
        else:
            if maximize:
                updates = optree.tree_map(lambda g: g.neg(), updates)
            if weight_decay != 0.0:
                updates = optree.tree_map(lambda g, p: g.add(p, alpha=weight_decay), updates, params)
        return updates, state

    return GradientTransformation(lambda params: EmptyState(), update_fn)
