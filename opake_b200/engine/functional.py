"""Stateless views of ``nn.Module`` for ``torch.func`` transforms, batch-dim adapters and the empty-batch collator.

Behaviour of packages/opake-engine/src/opake/api/engine/functional/__init__.py:15-360 and _collate.py:104-139:
``make_functional`` returns ``(fmodel, params)`` (tuple form) or ``(fmodel, trainable, frozen)`` (dict form split by
``requires_grad``); ``with_batch_dim`` lets a batched ``forward`` be called with one example under ``vmap`` by
unsqueezing the marked arguments and squeezing the result; ``empty_collate`` turns an empty Poisson draw into a
zero-length batch with the structure learned from the first non-empty one.
"""
from __future__ import annotations

import copy
import functools
import inspect
from collections.abc import Callable, Mapping
from typing import Any

import torch
from torch import nn

from .pytree import tree_map


def make_functional(mod: nn.Module, disable_autograd_tracking: bool = False, partition_trainable: bool = False):
    named = dict(mod.named_parameters())
    vals = {n: (p.detach() if disable_autograd_tracking else p) for n, p in named.items()}
    if partition_trainable:
        trainable = {n: vals[n] for n, p in named.items() if p.requires_grad}
        frozen = {n: vals[n] for n, p in named.items() if not p.requires_grad}

        def fmodel(params: Mapping[str, torch.Tensor], *args, **kwargs):
            return torch.func.functional_call(mod, params, args, kwargs)

        return fmodel, trainable, frozen
    names = list(vals)

    def fmodel_t(new_values, *args, **kwargs):
        return torch.func.functional_call(mod, dict(zip(names, new_values, strict=True)), args, kwargs)

    return fmodel_t, tuple(vals.values())


def _squeeze(out: Any) -> Any:
    if isinstance(out, torch.Tensor):
        return out.squeeze(0) if out.ndim > 0 else out
    if isinstance(out, Mapping):
        try:
            return type(out)({k: _squeeze(v) for k, v in out.items()})
        except Exception:
            return {k: _squeeze(v) for k, v in out.items()}
    if isinstance(out, tuple) and hasattr(out, "_fields"):
        return type(out)(*(_squeeze(v) for v in out))
    if isinstance(out, (list, tuple)):
        return type(out)(_squeeze(v) for v in out)
    if hasattr(out, "__dict__") and hasattr(out, "keys"):
        for k in list(out.keys()):
            out[k] = _squeeze(out[k])
    return out


def with_batch_dim(fn: Callable, batch_argnums=(), batch_kwargs=(), *, min_ndim: int | None = None) -> Callable:
    """Wrap ``fn`` (expects a leading batch dim) so it accepts single examples.

    ``batch_kwargs`` may be a sequence of names or a mapping ``name -> ndim threshold``. With ``min_ndim`` (or a
    threshold) only tensors of lower rank are unsqueezed and the output is squeezed only if something was.
    """
    if isinstance(batch_argnums, int):
        batch_argnums = (batch_argnums,)
    if not batch_argnums and not batch_kwargs:
        return fn
    thresholds = dict(batch_kwargs) if isinstance(batch_kwargs, Mapping) else {k: min_ndim for k in batch_kwargs}
    conditional = min_ndim is not None or any(v is not None for v in thresholds.values())
    positional_names: dict[int, str] = {}
    try:
        for i, (name, p) in enumerate(inspect.signature(fn).parameters.items()):
            if name in thresholds and p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD):
                positional_names[i] = name
    except (ValueError, TypeError):
        pass

    def needs(t: torch.Tensor, thr) -> bool:
        return True if thr is None else t.ndim < thr

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        changed = False
        a = list(args)
        for idx in sorted(positional_names, reverse=True):
            if idx < len(a) and positional_names[idx] not in kwargs:
                kwargs[positional_names[idx]] = a.pop(idx)

        def lift(x, thr=min_ndim):
            nonlocal changed
            if isinstance(x, torch.Tensor) and needs(x, thr):
                changed = True
                return x.unsqueeze(0)
            return x

        for i in batch_argnums:
            if i < len(a):
                a[i] = tree_map(lift, a[i])
        for name, thr in thresholds.items():
            v = kwargs.get(name)
            if isinstance(v, torch.Tensor) and needs(v, thr):
                changed = True
                kwargs[name] = v.unsqueeze(0)
        out = fn(*a, **kwargs)
        if (not conditional) or changed:
            out = _squeeze(out)
        return out

    wrapper._opake_batchified = True
    return wrapper


class _EmptyCollator:
    def __init__(self, collate_fn):
        self._fn, self._template = collate_fn, None

    def __call__(self, examples):
        if len(examples) == 0 and self._template is not None:
            return tree_map(lambda t: t[:0] if isinstance(t, torch.Tensor) else t, copy.deepcopy(self._template)) \
                if not isinstance(self._template, Mapping) else \
                type(self._template)({k: (v[:0] if isinstance(v, torch.Tensor) else v) for k, v in self._template.items()})
        out = self._fn(examples)
        if self._template is None:
            self._template = copy.deepcopy(out)
        return out


def empty_collate(collate_fn: Callable) -> Callable:
    return _EmptyCollator(collate_fn)


def under_differentiating_transform(when_compiling: bool = False) -> bool:
    """True when called inside ``torch.func.grad``/``vjp``/``jvp`` (so values must stay differentiable)."""
    try:
        from torch._C._functorch import TransformType, peek_interpreter_stack

        interp = peek_interpreter_stack()
        if interp is None:
            return False
        return interp.key() in (TransformType.Grad, TransformType.Jvp)
    except Exception:
        return False


__all__ = ["make_functional", "with_batch_dim", "empty_collate", "under_differentiating_transform"]
