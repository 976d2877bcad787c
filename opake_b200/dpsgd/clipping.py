"""Clipping transforms of the DP-SGD package: re-exports of the engine's fixed / AUTO-S / per-group clipping and the
quantile-tracking adaptive clipping of Andrew et al. (2021).

Adaptive rule (packages/opake-dpsgd/src/opake/api/dpsgd/clipping/_adaptive.py:31-675): after each step the noisy
clipped fraction ``rho = 0.5 + (num_clipped - B/2) / E[B] + N(0, sigma_b^2)`` drives a geometric update
``C <- clamp(C * exp(eta * (rho - gamma)), Cmin, Cmax)``; the noise draw for step ``t`` uses
``fold_in(key, "opake.dpsgd.adaptive_clipping", t[, group_index])``. The state carries local counts so that data-parallel
ranks can sum them and recompute the same next threshold.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch

from ..base.exceptions import ConfigurationError
from ..engine.clipping.auto import AutoClipState, auto_clipped_fun, auto_clipped_grad  # noqa: F401
from ..engine.clipping.core import (ClippedGradAux, ClippingStats, FixedClipState, _identity, _RuntimeClipState,  # noqa: F401
                                    _tuple, batch_size_from_args, clipped_fun, clipped_grad)
from ..engine.clipping.cuda_graph import CudaGraphChunkCompiler  # noqa: F401
from ..engine.clipping.per_group import per_group  # noqa: F401
from ..engine.pytree import tree_map
from ..engine.random import RngKey, fold_in, generator_from_key
from ..engine.types import ClipState, PerGroup, SecondMomentClippingOutput, clipped

ADAPTIVE_CLIPPING_STREAM_FOLD = "opake.dpsgd.adaptive_clipping"


@dataclass(frozen=True)
class AdaptiveClippedGradAux(ClippedGradAux):
    pass


@dataclass(frozen=True)
class AdaptiveClipState(ClipState):
    _current_clipping_norm: float | PerGroup
    _next_clipping_norm: float | PerGroup
    _step: int
    _rng_key: RngKey
    _fraction_noise_std: float
    _expected_batch_size: float
    _learning_rate: float
    _target_quantile: float
    _clipping_norm_min: float
    _clipping_norm_max: float
    _num_clipped: float | dict
    _batch_size: float

    def __post_init__(self):
        nxt = self._next_clipping_norm
        if isinstance(nxt, PerGroup):
            for g, v in nxt.values.items():
                if v <= 0:
                    raise ConfigurationError(f"next_clipping_norm must be positive for all groups, got {v} for group '{g}'")
        elif nxt <= 0:
            raise ConfigurationError(f"next_clipping_norm must be positive, got {nxt}")
        if self._expected_batch_size <= 0:
            raise ConfigurationError(f"expected_batch_size must be positive, got {self._expected_batch_size}")
        if self._fraction_noise_std <= 0:
            raise ConfigurationError(f"fraction_noise_std must be > 0, got {self._fraction_noise_std}")

    @property
    def clipping_norm(self):
        """Threshold that the next call will clip with."""
        return self._next_clipping_norm


def noisy_clipping_rate(num_clipped: float, batch_size: float, *, expected_batch_size: float, key: RngKey, step: int,
                        fraction_noise_std: float, group_index: int | None = None) -> float:
    stream = (ADAPTIVE_CLIPPING_STREAM_FOLD, step) + (() if group_index is None else (group_index,))
    z = torch.randn(1, generator=generator_from_key(fold_in(key, *stream))).item()
    return 0.5 + (num_clipped - batch_size / 2) / expected_batch_size + z * fraction_noise_std


def next_threshold(state: AdaptiveClipState, base, num_clipped, batch_size: float, step: int):
    def one(bound: float, count: float, gi=None) -> float:
        rho = noisy_clipping_rate(count, batch_size, expected_batch_size=state._expected_batch_size, key=state._rng_key,
                                  step=step, fraction_noise_std=state._fraction_noise_std, group_index=gi)
        f = torch.exp(torch.tensor(state._learning_rate * (rho - state._target_quantile))).item()
        return float(max(state._clipping_norm_min, min(state._clipping_norm_max, bound * f)))

    if isinstance(base, PerGroup):
        return PerGroup(base.groups, {n: one(base.values[n], num_clipped[n], i) for i, n in enumerate(sorted(base.values))})
    return one(base, num_clipped)


def adaptive_clipped_grad(loss_fn, argnums=0, has_aux=False, *, initial_clipping_norm=0.1, target_quantile=0.5,
                          learning_rate=0.2, clipping_norm_min=0.01, clipping_norm_max=100.0, fraction_noise_std=0.05,
                          expected_batch_size=None, key: RngKey, return_aux=False, return_stats=False,
                          pre_clipping_transform=_identity, **clipped_grad_kwargs):
    if return_aux and return_stats:
        raise ConfigurationError("return_stats cannot be combined with return_aux=True")
    normalize_by = clipped_grad_kwargs.get("normalize_by", 1.0)
    if expected_batch_size is None:
        expected_batch_size = clipped_grad_kwargs.get("normalize_by")
    if expected_batch_size is None:
        raise ConfigurationError("expected_batch_size is required when normalize_by is omitted")
    if expected_batch_size <= 0:
        raise ConfigurationError(f"expected_batch_size must be positive, got {expected_batch_size}")
    if not 0 < target_quantile < 1:
        raise ConfigurationError(f"target_quantile must be in (0, 1), got {target_quantile}")
    second_moment = bool(clipped_grad_kwargs.get("second_moment", False))
    barg = _tuple(clipped_grad_kwargs.get("batch_argnums", 1))
    arg_t = _tuple(argnums)
    grouped = isinstance(initial_clipping_norm, PerGroup)
    zero_counts = (lambda: dict.fromkeys(sorted(initial_clipping_norm.values), 0.0) if grouped else 0.0)
    inner, _ = clipped_grad(loss_fn, argnums=argnums, has_aux=has_aux, clipping_norm=initial_clipping_norm,
                            return_aux=return_aux, return_stats=not return_aux,
                            pre_clipping_transform=pre_clipping_transform, **clipped_grad_kwargs)
    state0 = AdaptiveClipState(initial_clipping_norm, initial_clipping_norm, 0, key, float(fraction_noise_std),
                               float(expected_batch_size), float(learning_rate), float(target_quantile),
                               float(clipping_norm_min), float(clipping_norm_max), zero_counts(), 0.0)

    def advance(state, counts, B):
        return replace(state, _current_clipping_norm=state._next_clipping_norm,
                       _next_clipping_norm=next_threshold(state, state._next_clipping_norm, counts, float(B), state._step),
                       _step=state._step + 1, _num_clipped=counts, _batch_size=float(B))

    def grad_fn(*args, state: AdaptiveClipState, **kwargs):
        with torch.profiler.record_function("opake::adaptive_clipped_grad"):
            C = state._next_clipping_norm
            if batch_size_from_args(args, barg) == 0:
                picked = args[arg_t[0]] if isinstance(argnums, int) else tuple(args[i] for i in arg_t)
                dt = clipped_grad_kwargs.get("dtype")
                zeros = tree_map(lambda t: torch.zeros_like(t, dtype=dt or t.dtype) if isinstance(t, torch.Tensor) else t,
                                 pre_clipping_transform(picked))
                grads = clipped(zeros, max_norm=C / normalize_by)
                if second_moment:
                    grads = SecondMomentClippingOutput(grads, clipped(tree_map(torch.zeros_like, zeros),
                                                                      max_norm=(C * C) / normalize_by))
                new = advance(state, zero_counts(), 0.0)
                if return_aux:
                    e = torch.empty(0)
                    return (grads, AdaptiveClippedGradAux(e, e, e, None, None if grouped else 0.0)), new
                if return_stats:
                    z = zero_counts()
                    return (grads, ClippingStats(z, dict(z) if grouped else 0.0, 0)), new
                return grads, new
            (grads, extra), _ = inner(*args, state=_RuntimeClipState(C), **kwargs)
            if return_aux:
                B = extra.batch_size
                if grouped:
                    counts = {n: float((extra.group_norms[n] > C.values[n]).sum().item()) for n in sorted(C.values)}
                else:
                    counts = float((extra.grad_norms > C).sum().item())
            else:
                B, counts = extra.batch_size, extra.num_clipped
            new = advance(state, counts, B)
            if return_aux:
                return (grads, AdaptiveClippedGradAux(extra.loss_values, extra.grad_norms, extra.clipped_grad_norms,
                                                      extra.loss_aux, extra.clipping_rate, extra.batch_size,
                                                      extra.group_norms)), new
            if return_stats:
                return (grads, extra), new
            return grads, new

    return grad_fn, state0


def sync_adaptive_clip_state(state: AdaptiveClipState) -> AdaptiveClipState:
    """Data-parallel agreement: sum local counts over ranks, then recompute the next threshold from the totals
    (packages/opake-dpsgd/src/opake/api/dpsgd/clipping/_distributed.py:50-103)."""
    from ..engine import distributed as D

    if not D.is_distributed():
        return state
    D.assert_scalar_equal(state._step, name="AdaptiveClipState._step")
    B = D.reduce_scalar(float(state._batch_size), "sum")
    if isinstance(state._num_clipped, dict):
        counts = {k: D.reduce_scalar(float(v), "sum") for k, v in sorted(state._num_clipped.items())}
    else:
        counts = D.reduce_scalar(float(state._num_clipped), "sum")
    nxt = next_threshold(state, state._current_clipping_norm, counts, B, state._step - 1)
    return replace(state, _next_clipping_norm=nxt, _num_clipped=counts, _batch_size=B)


def _register():
    from ..engine import distributed as D

    D.register_sync_type(AdaptiveClipState, sync_adaptive_clip_state)
    D.register_sync_type(FixedClipState, lambda s: s)
    D.register_sync_type(AutoClipState, lambda s: s)
    # per-example aux outputs and clipping statistics: gathered / summed over the ranks by sync()
    from ..engine.clipping.core import ClippedFunAux
    from ..engine.clipping.distributed import sync_clipping_aux
    for aux_type in (ClippedGradAux, ClippedFunAux, ClippingStats):
        D.register_sync_type(aux_type, sync_clipping_aux)


_register()

__all__ = ["AdaptiveClipState", "AdaptiveClippedGradAux", "adaptive_clipped_grad", "auto_clipped_fun", "auto_clipped_grad",
           "clipped_fun", "clipped_grad", "per_group", "CudaGraphChunkCompiler", "ClippingStats", "FixedClipState",
           "AutoClipState", "sync_adaptive_clip_state"]
