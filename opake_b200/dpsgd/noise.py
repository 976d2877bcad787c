"""Gaussian mechanism: ``noise_fn(ClippedPytree, state) -> (NoisedPytree, state)``.

Semantics of packages/opake-dpsgd/src/opake/api/dpsgd/noise/_gaussian.py:58-345: the key of step ``t`` is
``fold_in(key, "opake.dpsgd.gaussian", t)``; ``sigma = noise_multiplier * max_norm`` (per-group: MSE-optimal
allocation); paired first/second-moment inputs use two sub-streams; the state is ``(_step_counter, _rng_key)``.

Two noise sources:

* ``backend="generator"`` — the reference's: ONE CPU ``torch.Generator`` seeded from the step key, consumed leaf by
  leaf in tree order, each draw copied to the leaf's device. Bit-compatible with the reference; default for CPU
  tensors.
* ``backend="philox"`` — the B200 one: counter-based Philox4x32-10 on the device, element ``e`` of the flattened tree
  (leaves concatenated in tree order) uses counter ``e // 4``. No host work, no H2D copy, and any sharding of the
  flattened tree draws the same global noise tensor, which is what lets the sharded engine add noise exactly once.
  Default for CUDA tensors. Statistically equivalent to the generator backend, not bitwise.
"""
from __future__ import annotations

import dataclasses

import torch

from ..base.exceptions import ConfigurationError, InputTypeError
from ..base.serialization import register_serializer
from ..engine.noise_allocation import (PAIRED_FIRST_STREAM_FOLD, PAIRED_SECOND_STREAM_FOLD, per_group_noise_stddev,
                                       resolve_paired_clipped)
from ..engine.pytree import tree_flatten_with_paths, tree_unflatten
from ..engine.random import RngKey, fold_in, generator_from_key
from ..engine.types import (ClippedPytree, NoisedPytree, NoiseState, PerGroup, SecondMomentClippingOutput,
                            SecondMomentNoiseOutput)

GAUSSIAN_STREAM_FOLD = "opake.dpsgd.gaussian"
_DTYPES = {torch.float16, torch.bfloat16, torch.float32, torch.float64}


@dataclasses.dataclass(frozen=True)
class GaussianNoiseState(NoiseState):
    _step_counter: int
    _rng_key: RngKey


def _check_std(std) -> None:
    if isinstance(std, PerGroup):
        for g, v in std.values.items():
            if v < 0:
                raise ConfigurationError(f"noise standard deviation must be non-negative for all groups, got {v} for group '{g}'")
    elif std < 0:
        raise ConfigurationError(f"noise standard deviation must be non-negative, got {std}")


def _philox_add(center: torch.Tensor, std: float, seed: int, offset: int, compute_dtype) -> torch.Tensor:
    if center.is_cuda:
        from ..ops import kernels as K

        z = K.philox_normal_(torch.empty(center.numel(), dtype=torch.float32, device=center.device), seed, 0,
                             offset=offset, sigma=1.0)
    else:
        from ..ops.philox_ref import normal

        z = torch.from_numpy(normal(center.numel(), seed, 0, offset=offset))
    out = center.to(compute_dtype) + std * z.view(center.shape).to(compute_dtype)
    return out.to(center.dtype)


def add_gaussian_noise_tree(tree, stddev, step_key: RngKey, *, compute_dtype=torch.float32, backend: str = "auto"):
    """``leaf + N(0, std^2)`` for every tensor leaf, in tree order."""
    _check_std(stddev)
    paths, leaves, td = tree_flatten_with_paths(tree)
    gen = None
    out, offset = [], 0
    for path, leaf in zip(paths, leaves):
        if not isinstance(leaf, torch.Tensor):
            if isinstance(stddev, PerGroup):
                raise InputTypeError(f"gaussian_noise with PerGroup stddev expects tensor leaves; got "
                                     f"{type(leaf).__name__} at path {path!r}.")
            out.append(leaf)
            continue
        std = stddev.for_path(path) if isinstance(stddev, PerGroup) else float(stddev)
        mode = backend if backend != "auto" else ("philox" if leaf.is_cuda else "generator")
        if mode == "generator":
            gen = gen or generator_from_key(step_key)
            if std == 0:
                out.append(leaf)
            else:
                z = torch.randn(leaf.shape, dtype=compute_dtype, generator=gen).to(leaf.device)
                out.append((leaf.to(compute_dtype) + std * z).to(leaf.dtype))
        elif mode == "philox":
            out.append(leaf if std == 0 else _philox_add(leaf, std, step_key.seed, offset, compute_dtype))
            offset += (leaf.numel() + 3) // 4 * 4
        else:
            raise ConfigurationError(f"unknown noise backend {backend!r}")
    return tree_unflatten(td, out)


def gaussian_noise(*, noise_multiplier: float, key: RngKey, compute_dtype: torch.dtype = torch.float32,
                   backend: str = "auto"):
    if noise_multiplier is None:
        raise ConfigurationError("gaussian_noise() requires noise_multiplier.")
    nm = float(noise_multiplier)
    if nm < 0:
        raise ConfigurationError(f"noise_multiplier must be non-negative, got {noise_multiplier}")
    if not isinstance(compute_dtype, torch.dtype):
        raise InputTypeError(f"compute_dtype must be torch.dtype, got {type(compute_dtype).__name__}")
    if compute_dtype not in _DTYPES:
        raise ConfigurationError("compute_dtype must be one of torch.float16, torch.bfloat16, torch.float32, or "
                                 f"torch.float64; got {compute_dtype}.")
    if not isinstance(key, RngKey):
        raise InputTypeError(f"key must be RngKey, got {type(key)}")

    def stddev_of(c: ClippedPytree):
        if isinstance(c.max_norm, PerGroup):
            return per_group_noise_stddev(c.max_norm, nm)
        s = 0.0 if nm == 0.0 else nm * c.max_norm
        _check_std(s)
        return s

    def noise_fn(grads, st: GaussianNoiseState):
        with torch.profiler.record_function("opake::gaussian_noise"):
            nxt = GaussianNoiseState(st._step_counter + 1, st._rng_key)
            if isinstance(grads, SecondMomentClippingOutput):
                a, b, s1, s2 = resolve_paired_clipped(grads, noise_multiplier=nm)
                k1 = fold_in(st._rng_key, GAUSSIAN_STREAM_FOLD, PAIRED_FIRST_STREAM_FOLD, st._step_counter)
                k2 = fold_in(st._rng_key, GAUSSIAN_STREAM_FOLD, PAIRED_SECOND_STREAM_FOLD, st._step_counter)
                n1 = add_gaussian_noise_tree(a.pytree, s1, k1, compute_dtype=compute_dtype, backend=backend)
                n2 = add_gaussian_noise_tree(b.pytree, s2, k2, compute_dtype=compute_dtype, backend=backend)
                return SecondMomentNoiseOutput(NoisedPytree(n1, a.max_norm, s1), NoisedPytree(n2, b.max_norm, s2)), nxt
            if isinstance(grads, NoisedPytree):
                raise InputTypeError("gaussian_noise expects ClippedPytree inputs, not NoisedPytree values that have "
                                     "already passed through a noise mechanism.")
            if not isinstance(grads, ClippedPytree):
                raise InputTypeError("gaussian_noise expects ClippedPytree inputs. Wrap manual values with "
                                     "opake.types.clipped(...).")
            std = stddev_of(grads)
            k = fold_in(st._rng_key, GAUSSIAN_STREAM_FOLD, st._step_counter)
            noisy = add_gaussian_noise_tree(grads.pytree, std, k, compute_dtype=compute_dtype, backend=backend)
            return NoisedPytree(noisy, grads.max_norm, std), nxt

    return noise_fn, GaussianNoiseState(0, key)


def sync_gaussian_noise_state(state: GaussianNoiseState) -> GaussianNoiseState:
    """Every rank must hold the same key and step (packages/opake-dpsgd/.../noise/_distributed.py:25-50)."""
    from ..engine import distributed as D

    D.assert_string_equal(str(state._rng_key.seed), name="GaussianNoiseState._rng_key.seed")
    D.assert_scalar_equal(state._step_counter, name="GaussianNoiseState._step_counter")
    return state


def _register():
    from ..engine import distributed as D

    D.register_sync_type(GaussianNoiseState, sync_gaussian_noise_state)


_register()

__all__ = ["GAUSSIAN_STREAM_FOLD", "GaussianNoiseState", "gaussian_noise", "add_gaussian_noise_tree",
           "sync_gaussian_noise_state"]
