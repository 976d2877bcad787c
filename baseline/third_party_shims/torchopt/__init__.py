"""Minimal stand-in for the ``torchopt`` package: only the functional-optimizer surface the reference imports
(``base.GradientTransformation``, ``chain``, ``apply_updates``, ``sgd``, ``adamw``, ``transform.add_decayed_weights``,
``alias.utils.scale_by_neg_lr``), with the documented semantics of the real library (in-place by default)."""
from __future__ import annotations

from typing import Any, Callable

import optree

from . import alias, base, transform
from .alias.utils import flip_sign_and_add_weight_decay, scale_by_neg_lr
from .base import GradientTransformation, chain

__version__ = "0.7.3+standin"


def apply_updates(params: Any, updates: Any, *, inplace: bool = True) -> Any:
    """``params + updates`` leaf by leaf; in place on ``param.data`` unless ``inplace=False``."""
    if inplace:
        def f(p, u):
            if u is not None:
                p.data.add_(u)
            return p

        optree.tree_map(f, params, updates)
        return params
    return optree.tree_map(lambda p, u: p.add(u) if u is not None else p, params, updates)


def sgd(lr: float | Callable, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False, *,
        moment_requires_grad: bool = False, maximize: bool = False) -> GradientTransformation:
    if not momentum >= 0.0:
        raise ValueError(f"Invalid momentum value: {momentum}")
    if nesterov and (momentum <= 0.0 or dampening != 0.0):
        raise ValueError("Nesterov momentum requires a momentum and zero dampening")
    return chain(flip_sign_and_add_weight_decay(weight_decay=weight_decay, maximize=maximize),
                 transform.trace(momentum=momentum, dampening=dampening, nesterov=nesterov, moment_requires_grad=moment_requires_grad),
                 scale_by_neg_lr(lr))


def adamw(lr: float | Callable = 1e-3, betas: tuple = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2, *, eps_root: float = 0.0,
          mask: Any = None, moment_requires_grad: bool = False, maximize: bool = False, use_accelerated_op: bool = False) -> GradientTransformation:
    return chain(flip_sign_and_add_weight_decay(weight_decay=0.0, maximize=maximize),
                 transform.scale_by_adam(b1=betas[0], b2=betas[1], eps=eps, eps_root=eps_root),
                 transform.add_decayed_weights(weight_decay=weight_decay, mask=mask),
                 scale_by_neg_lr(lr))


__all__ = ["GradientTransformation", "alias", "apply_updates", "adamw", "base", "chain", "sgd", "transform"]
