"""Per-example clipping transforms: ``clipped_fun`` (any per-example function) and ``clipped_grad`` (its gradient).

API and return conventions follow packages/opake-engine/src/opake/api/engine/clipping/_clipped_fun.py:492-944 and
_clipped_grad.py:86-362: factories return ``(fn, FixedClipState)``; ``fn(*args, state=...)`` returns
``(ClippedPytree, state)`` or ``((ClippedPytree, aux_or_stats), state)``; the output is the *sum* of clipped
per-example values divided by ``normalize_by`` with ``max_norm = clipping_norm / normalize_by``; empty batches give
zeros with the same sensitivity.

Execution: the batch is cut into micro-batches; each micro-batch is evaluated with ``torch.func.vmap`` (optionally
through a chunk compiler such as :class:`CudaGraphChunkCompiler`), clipped with the conservative arithmetic of
:mod:`.numerics` (or the fused CUDA clip-sum backend when one is registered) and added to an fp32 accumulator. For
transformer training on B200 the native runtimes (:mod:`opake_b200.models`) bypass vmap entirely; this module is the
general-purpose path for arbitrary ``loss_fn``.
"""
from __future__ import annotations

import contextlib
from collections.abc import Callable
from dataclasses import dataclass
from typing import Any

import torch
from torch.func import grad_and_value, vmap

from ...base.exceptions import ConfigurationError, InputTypeError
from ..pytree import param_path_display, tree_flatten_with_paths, tree_map, tree_unflatten
from ..types import ClippedPytree, ClipState, PerGroup, SecondMomentClippingOutput, clipped
from . import numerics as N
from .kernel_backend import get_fused_clip_backend
from .streaming import resolve_stream_impl, stream_clip_and_sum


@dataclass(frozen=True)
class FixedClipState(ClipState):
    """Marker state of fixed clipping (the threshold lives in ``ClippedPytree.max_norm``)."""


@dataclass(frozen=True)
class _RuntimeClipState(FixedClipState):
    clipping_norm: Any = None


@dataclass(frozen=True)
class ClippedFunAux:
    values: Any | None = None
    norms: Any | None = None
    clipped_norms: Any | None = None
    value_aux: Any | None = None
    clipping_rate: float | None = None
    batch_size: int = 0
    group_norms: dict | None = None


@dataclass(frozen=True)
class ClippingStats:
    num_clipped: Any
    clipping_rate: Any
    batch_size: int = 0


@dataclass(frozen=True)
class ClippedGradAux:
    loss_values: Any | None = None
    grad_norms: Any | None = None
    clipped_grad_norms: Any | None = None
    loss_aux: Any | None = None
    clipping_rate: float | None = None
    batch_size: int = 0
    group_norms: dict | None = None


@dataclass(frozen=True)
class _BuiltinScale:
    kind: str = "fixed"      # "fixed" | "auto"
    gamma: float = 0.01


def _tuple(x) -> tuple[int, ...]:
    return (x,) if isinstance(x, int) else tuple(x)


def batch_size_from_args(args, batch_argnums: tuple[int, ...]) -> int:
    for i in batch_argnums:
        leaves = [l for l in tree_flatten_with_paths(args[i])[1] if isinstance(l, torch.Tensor)]
        if leaves:
            return int(leaves[0].shape[0])
    raise ConfigurationError("no batched tensor argument found")


def _slice_args(args, batch_argnums, lo, hi):
    out = list(args)
    for i in batch_argnums:
        out[i] = tree_map(lambda t: t[lo:hi] if isinstance(t, torch.Tensor) else t, args[i])
    return tuple(out)


def _group_of(paths, clipping_norm: PerGroup):
    names = []
    for p in paths:
        if p not in clipping_norm.groups:
            raise ConfigurationError(f"leaf {param_path_display(p)!r} has no clipping group")
        names.append(clipping_norm.groups[p])
    return names


class _Accumulator:
    """fp32 running sum of clipped micro-batch sums (plus the optional squared stream)."""

    def __init__(self):
        self.sum = None
        self.sq = None

    def add(self, leaves, sq_leaves=None):
        if self.sum is None:
            self.sum = [l.clone() for l in leaves]
            self.sq = [l.clone() for l in sq_leaves] if sq_leaves is not None else None
        else:
            for a, l in zip(self.sum, leaves):
                a.add_(l)
            if sq_leaves is not None:
                for a, l in zip(self.sq, sq_leaves):
                    a.add_(l)


def clipped_fun(fun: Callable, has_aux: bool = False, *, batch_argnums=0, clipping_norm=1.0, normalize_by: float = 1.0,
                return_aux: bool = False, return_stats: bool = False, second_moment: bool = False,
                microbatch_size: int | None = None, dtype: torch.dtype | None = None,
                compute_dtype: torch.dtype | None = None, _scale_fn=None, _builtin_scale: _BuiltinScale | None = None,
                _chunk_compiler=None):
    """Clip ``fun``'s per-example outputs to ``clipping_norm`` and sum them over the batch."""
    if return_aux and return_stats:
        raise ConfigurationError("return_stats cannot be combined with return_aux=True")
    if microbatch_size is not None and microbatch_size < 1:
        raise ConfigurationError(f"microbatch_size must be >= 1, got {microbatch_size}")
    if not (normalize_by > 0):
        raise ConfigurationError(f"normalize_by must be positive, got {normalize_by}")
    bargs = _tuple(batch_argnums)
    builtin = _builtin_scale or _BuiltinScale()
    per_group = isinstance(clipping_norm, PerGroup)

    def chunk_values(args, kwargs):
        in_dims = tuple(0 if i in bargs else None for i in range(len(args)))
        f = (lambda *a: fun(*a, **kwargs))
        return vmap(f, in_dims=in_dims, randomness="different")(*args)

    run_chunk = _chunk_compiler.wrap(chunk_values) if _chunk_compiler is not None else chunk_values

    def clip_chunk(values, norm_value):
        paths, leaves, td = tree_flatten_with_paths(values)
        leaves = [N.sanitize(l) for l in leaves]
        if not leaves:
            return td, [], None, None, None, None, None
        dev = leaves[0].device
        sqd = compute_dtype if compute_dtype is not None else N.sq_dtype_for(dev)
        B = leaves[0].shape[0]
        group_norms = None
        if per_group:
            names = _group_of(paths, norm_value)
            factors = [None] * len(leaves)
            group_norms, masks = {}, {}
            for gname in sorted(set(names)):
                idx = [i for i, n in enumerate(names) if n == gname]
                sq = sum(N.per_example_sq(leaves[i], sqd) for i in idx)
                fs, norms, mask = N.clip_factors(sq, norm_value.values[gname], [leaves[i] for i in idx],
                                                 auto=builtin.kind == "auto", gamma=builtin.gamma)
                for i, f in zip(idx, fs):
                    factors[i] = f
                group_norms[gname], masks[gname] = norms, mask
            norms = torch.sqrt(sum(v * v for v in group_norms.values()))
            mask = masks
        else:
            impl = resolve_stream_impl(leaves, norm_value, scale_fn=_scale_fn, builtin_kind=builtin.kind, second_moment=second_moment,
                                       compute_dtype=compute_dtype)
            if impl == "fused":
                # CUDA: two multi-tensor kernels replace the per-leaf square / scale / sum passes
                sums, norms, mask, cn = get_fused_clip_backend().fused_clip_sum(leaves, float(norm_value), with_postsq=return_aux)
                return td, sums, None, norms, mask, cn, None
            # portable two-pass streaming path: no scaled copy of the whole per-example gradient
            sums, sq_sums, norms, mask, cn = stream_clip_and_sum(leaves, norm_value, scale_fn=_scale_fn, auto=builtin.kind == "auto",
                                                                 gamma=builtin.gamma, second_moment=second_moment,
                                                                 compute_dtype=compute_dtype, with_postsq=return_aux)
            return td, sums, sq_sums, norms, mask, cn, None
        scaled = [N.scale_leaf(l, f) for l, f in zip(leaves, factors)]
        sums = [s.sum(0, dtype=N.acc_dtype_of(s.dtype)) for s in scaled]
        sq_sums = None
        if second_moment:
            sq_sums = [(s.to(N.acc_dtype_of(s.dtype)) ** 2).sum(0) for s in scaled]
        clipped_norms = None
        if return_aux:
            clipped_norms = torch.sqrt(sum(N.per_example_sq(s, sqd) for s in scaled))
        return td, sums, sq_sums, norms, mask, clipped_norms, group_norms

    def fn(*args, state: FixedClipState, **kwargs):
        norm_value = state.clipping_norm if isinstance(state, _RuntimeClipState) and state.clipping_norm is not None \
            else clipping_norm
        B = batch_size_from_args(args, bargs)
        step = microbatch_size or B
        acc = _Accumulator()
        td = None
        all_norms, all_clipped, all_values, all_aux, all_gn = [], [], [], [], []
        n_clipped = {} if per_group else 0.0
        for lo in range(0, B, step):
            cargs = _slice_args(args, bargs, lo, min(B, lo + step))
            out = run_chunk(cargs, kwargs)
            if has_aux:
                values, aux = out
            else:
                values, aux = out, None
            td, sums, sq_sums, norms, mask, cn, gn = clip_chunk(values, norm_value)
            acc.add(sums, sq_sums)
            if per_group:
                for g, m in mask.items():
                    n_clipped[g] = n_clipped.get(g, 0.0) + float(m.sum())
            else:
                n_clipped += float(mask.sum()) if mask is not None else 0.0
            if return_aux:
                all_norms.append(norms)
                all_clipped.append(cn)
                all_gn.append(gn)
                if aux is not None:
                    all_values.append(aux.get("values") if isinstance(aux, dict) else None)
                    all_aux.append(aux.get("value_aux") if isinstance(aux, dict) else aux)
        inv = 1.0 / normalize_by

        def finish(leaves):
            outl = []
            for l in leaves:
                o = l * inv
                outl.append(o.to(dtype) if dtype is not None else o)
            return tree_unflatten(td, outl)

        max_norm = norm_value / normalize_by if not isinstance(norm_value, PerGroup) else norm_value / normalize_by
        result = clipped(finish(acc.sum), max_norm=max_norm)
        if second_moment:
            sq_norm = (norm_value * norm_value) / normalize_by
            result = SecondMomentClippingOutput(result, clipped(finish(acc.sq), max_norm=sq_norm))
        if return_stats:
            rate = ({g: c / B for g, c in n_clipped.items()} if per_group else n_clipped / B) if B else None
            return (result, ClippingStats(n_clipped, rate, B)), state
        if return_aux:
            cat = (lambda xs: torch.cat(xs) if xs and all(x is not None for x in xs) else None)

            def cat_tree(xs):
                xs = [x for x in xs if x is not None]
                if not xs:
                    return None
                return tree_map(lambda *ts: torch.cat(ts) if isinstance(ts[0], torch.Tensor) else ts[0], *xs)

            gn = None
            if per_group and all_gn:
                gn = {g: torch.cat([d[g] for d in all_gn]) for g in all_gn[0]}
            rate = None if per_group else (n_clipped / B if B else 0.0)
            aux_out = ClippedFunAux(values=cat_tree(all_values), norms=cat(all_norms), clipped_norms=cat(all_clipped),
                                    value_aux=cat_tree(all_aux), clipping_rate=rate, batch_size=B, group_norms=gn)
            return (result, aux_out), state
        return result, state

    return fn, FixedClipState()


def _identity(x):
    return x


def clipped_grad(loss_fn: Callable, argnums=0, has_aux: bool = False, *, clipping_norm, normalize_by: float = 1.0,
                 batch_argnums=1, return_aux: bool = False, return_stats: bool = False, second_moment: bool = False,
                 pre_clipping_transform: Callable = _identity, microbatch_size: int | None = None,
                 dtype: torch.dtype | None = None, compute_dtype: torch.dtype | None = None, _scale_fn=None,
                 _builtin_scale=None, _chunk_compiler=None):
    """Sum of clipped per-example gradients of ``loss_fn`` (a function of ONE example) divided by ``normalize_by``."""
    if return_aux and return_stats:
        raise ConfigurationError("return_stats cannot be combined with return_aux=True")
    arg_t, barg_t = _tuple(argnums), _tuple(batch_argnums)
    if set(arg_t) & set(barg_t):
        raise ConfigurationError("argnums and batch_argnums must be disjoint")
    gv = grad_and_value(loss_fn, argnums=argnums, has_aux=has_aux)

    def per_example(*args, **kwargs):
        if has_aux:
            grad, (value, aux) = gv(*args, **kwargs)
        else:
            (grad, value), aux = gv(*args, **kwargs), None
        g = pre_clipping_transform(grad)
        if return_aux:
            d = {"values": value}
            if has_aux:
                d["value_aux"] = aux
            return g, d
        return g

    inner, state0 = clipped_fun(per_example, has_aux=return_aux, batch_argnums=batch_argnums,
                                clipping_norm=clipping_norm, normalize_by=normalize_by, return_aux=return_aux,
                                return_stats=return_stats, second_moment=second_moment,
                                microbatch_size=microbatch_size, dtype=dtype, compute_dtype=compute_dtype,
                                _scale_fn=_scale_fn, _builtin_scale=_builtin_scale, _chunk_compiler=_chunk_compiler)
    out_norm = clipping_norm / normalize_by

    def empty(args, state):
        picked = args[arg_t[0]] if isinstance(argnums, int) else tuple(args[i] for i in arg_t)
        zeros = tree_map(lambda t: torch.zeros_like(t, dtype=dtype or t.dtype) if isinstance(t, torch.Tensor) else t,
                         pre_clipping_transform(picked))
        grads = clipped(zeros, max_norm=out_norm)
        if second_moment:
            grads = SecondMomentClippingOutput(grads, clipped(tree_map(torch.zeros_like, zeros),
                                                              max_norm=(clipping_norm * clipping_norm) / normalize_by))
        if return_aux:
            e = torch.empty(0)
            return (grads, ClippedGradAux(e, e, e, None, None if isinstance(clipping_norm, PerGroup) else 0.0, 0)), state
        if return_stats:
            if isinstance(clipping_norm, PerGroup):
                names = sorted(clipping_norm.values)
                return (grads, ClippingStats(dict.fromkeys(names, 0.0), dict.fromkeys(names, 0.0), 0)), state
            return (grads, ClippingStats(0.0, 0.0, 0)), state
        return grads, state

    def grad_fn(*args, state, **kwargs):
        if batch_size_from_args(args, barg_t) == 0:
            return empty(args, state)
        ctx = torch.no_grad()
        with torch.profiler.record_function("opake::clipped_grad"), ctx:
            out, st = inner(*args, state=state, **kwargs)
        if return_aux:
            g, a = out
            return (g, ClippedGradAux(a.values, a.norms, a.clipped_norms, a.value_aux, a.clipping_rate, a.batch_size,
                                      a.group_norms)), st
        return out, st

    return grad_fn, state0


__all__ = ["ClippedFunAux", "ClippedGradAux", "ClippingStats", "FixedClipState", "clipped_fun", "clipped_grad",
           "batch_size_from_args"]
