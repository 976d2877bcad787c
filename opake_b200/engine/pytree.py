"""Pytree helpers on ``torch.utils._pytree`` (paths are tuples of dict keys / sequence indices).

Mirrors the surface of packages/opake-engine/src/opake/api/engine/pytree.py:39-480 (``ParamPath``,
``tree_flatten_with_paths``, ``tree_map``, ``partition``, ``merge``, ``global_norm``); dict traversal is in sorted key
order like optree's, so per-group bookkeeping keyed by path is stable.
"""
from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
import torch.utils._pytree as _pt

from ..base.exceptions import ConfigurationError, InputTypeError

ParamPath = tuple  # tuple[str | int, ...]
_RAW_ERR = ("Tensor-leaf operations require raw tensor pytrees. Pass a single-stream wrapper's `.pytree`; for paired "
            "output, select a stream and pass that stream's `.pytree`.")


def param_path(path) -> ParamPath:
    if isinstance(path, str):
        return (path,)
    out = []
    for part in path:
        if isinstance(part, (str, int)):
            out.append(part)
        else:
            raise InputTypeError(f"ParamPath components must be str or int; got {type(part).__name__}")
    return tuple(out)


def param_path_display(path: ParamPath) -> str:
    return ".".join(str(p) for p in path)


def _is_leaf(x: Any) -> bool:
    return not isinstance(x, (dict, list, tuple)) or (isinstance(x, tuple) and hasattr(x, "_fields") and False)


def _walk(tree: Any, path: tuple, paths: list, leaves: list) -> Any:
    """Flatten with sorted dict keys; returns a structure skeleton used by :func:`tree_unflatten`."""
    if isinstance(tree, dict):
        keys = sorted(tree.keys(), key=lambda k: (str(type(k)), k))
        return ("dict", type(tree), keys, [_walk(tree[k], (*path, k), paths, leaves) for k in keys])
    if isinstance(tree, tuple) and hasattr(tree, "_fields"):
        return ("namedtuple", type(tree), None, [_walk(v, (*path, i), paths, leaves) for i, v in enumerate(tree)])
    if isinstance(tree, (list, tuple)):
        return ("seq", type(tree), None, [_walk(v, (*path, i), paths, leaves) for i, v in enumerate(tree)])
    if tree is None:
        return ("none", None, None, [])
    paths.append(path)
    leaves.append(tree)
    return ("leaf", None, None, [])


class TreeDef:
    """Structure of a pytree (everything but the leaves)."""

    def __init__(self, skeleton, n):
        self.skeleton, self.num_leaves = skeleton, n

    def __eq__(self, other):
        return isinstance(other, TreeDef) and self.skeleton == other.skeleton

    def __hash__(self):
        return hash(repr(self.skeleton))

    def __repr__(self):
        return f"TreeDef({self.num_leaves} leaves)"


def tree_flatten_with_paths(tree: Any):
    paths, leaves = [], []
    sk = _walk(tree, (), paths, leaves)
    return paths, leaves, TreeDef(sk, len(leaves))


def tree_flatten(tree: Any):
    _, leaves, td = tree_flatten_with_paths(tree)
    return leaves, td


def _build(sk, it):
    kind, typ, keys, kids = sk
    if kind == "leaf":
        return next(it)
    if kind == "none":
        return None
    if kind == "dict":
        return typ((k, _build(c, it)) for k, c in zip(keys, kids)) if typ is not dict else {k: _build(c, it) for k, c in zip(keys, kids)}
    vals = [_build(c, it) for c in kids]
    if kind == "namedtuple":
        return typ(*vals)
    return typ(vals)


def tree_unflatten(treedef: TreeDef, leaves) -> Any:
    leaves = list(leaves)
    if len(leaves) != treedef.num_leaves:
        raise ConfigurationError(f"expected {treedef.num_leaves} leaves, got {len(leaves)}")
    return _build(treedef.skeleton, iter(leaves))


def tree_structure(tree: Any) -> TreeDef:
    return tree_flatten(tree)[1]


def tree_leaves(tree: Any) -> list[torch.Tensor]:
    flat, _ = tree_flatten(tree)
    tensors = [x for x in flat if isinstance(x, torch.Tensor)]
    if len(tensors) != len(flat):
        from .types import ClippedPytree

        if any(isinstance(x, ClippedPytree) for x in flat):
            raise InputTypeError(_RAW_ERR)
    return tensors


def tree_map(fn: Callable[..., Any], *trees: Any) -> Any:
    leaves0, td = tree_flatten(trees[0])
    rest = []
    for t in trees[1:]:
        lv, td2 = tree_flatten(t)
        if td2 != td:
            raise ConfigurationError("tree_map: trees have different structures")
        rest.append(lv)
    return tree_unflatten(td, [fn(*xs) for xs in zip(leaves0, *rest)])


def tree_map_with_path(fn: Callable[[ParamPath, Any], Any], tree: Any) -> Any:
    paths, leaves, td = tree_flatten_with_paths(tree)
    return tree_unflatten(td, [fn(p, x) for p, x in zip(paths, leaves)])


def partition(predicate: Callable[[tuple, Any], bool], tree: Any):
    """Split into (matching, rest); branches left without leaves disappear (used for LoRA / frozen splits)."""

    def rec(path, sub):
        if isinstance(sub, dict):
            yes, no = {}, {}
            for k, v in sub.items():
                a, b = rec((*path, k), v)
                if a is not None:
                    yes[k] = a
                if b is not None:
                    no[k] = b
            return (yes or None), (no or None)
        if isinstance(sub, (list, tuple)):
            pairs = [rec((*path, i), v) for i, v in enumerate(sub)]
            ys, ns = [p[0] for p in pairs], [p[1] for p in pairs]
            return (type(sub)(ys) if any(x is not None for x in ys) else None,
                    type(sub)(ns) if any(x is not None for x in ns) else None)
        return (sub, None) if predicate(path, sub) else (None, sub)

    yes, no = rec((), tree)
    empty = (lambda: {} if isinstance(tree, dict) else type(tree)())
    return (yes if yes is not None else empty()), (no if no is not None else empty())


def _merge2(a, b):
    if a is None:
        return b
    if b is None:
        return a
    if isinstance(a, dict) and isinstance(b, dict):
        out = dict(a)
        for k, v in b.items():
            out[k] = _merge2(out[k], v) if k in out else v
        return out
    if isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        if len(a) != len(b):
            raise ConfigurationError(f"Cannot merge sequences of different lengths: {len(a)} vs {len(b)}")
        return type(a)([_merge2(x, y) for x, y in zip(a, b)])
    return b


def merge(*trees: Any) -> Any:
    trees = [t for t in trees if t is not None]
    if not trees:
        return {}
    out = trees[0]
    for t in trees[1:]:
        out = _merge2(out, t)
    return out


def global_norm(tree: Any, *, compute_dtype: torch.dtype | None = None) -> torch.Tensor:
    from .types import ClippedPytree, SecondMomentClippingOutput, SecondMomentNoiseOutput

    if isinstance(tree, (ClippedPytree, SecondMomentClippingOutput, SecondMomentNoiseOutput)):
        raise InputTypeError(_RAW_ERR)
    if compute_dtype is not None and not compute_dtype.is_floating_point:
        raise InputTypeError(f"compute_dtype must be a real floating-point dtype, got {compute_dtype!r}.")
    leaves = tree_leaves(tree)
    if not leaves:
        return torch.tensor(0.0, dtype=compute_dtype or torch.float32)
    acc = compute_dtype
    if acc is None:
        acc = torch.float32
        for t in leaves:
            dt = t.real.dtype if t.is_complex() else t.dtype
            if dt.is_floating_point:
                acc = torch.promote_types(acc, dt)
    total = torch.zeros((), device=leaves[0].device, dtype=acc)
    for t in leaves:
        parts = (t.real, t.imag) if t.is_complex() else (t,)
        for p in parts:
            x = p.to(acc)
            total = total + (x * x).sum(dtype=acc)
    return torch.sqrt(total)


__all__ = ["ParamPath", "param_path", "param_path_display", "tree_flatten_with_paths", "tree_flatten", "tree_unflatten",
           "tree_structure", "tree_leaves", "tree_map", "tree_map_with_path", "partition", "merge", "global_norm",
           "TreeDef"]
