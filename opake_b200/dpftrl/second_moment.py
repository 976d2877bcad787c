"""Paired first/second-moment correlated noise (packages/opake-dpftrl/src/opake/api/dpftrl/noise/_second_moment.py:
38-200): two independent matrix-factorisation streams keyed by ``opake.dpftrl.second_moment.first/second`` whose joint
allocation gives the PLD of a single mechanism at the calibrated noise multiplier."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any

import torch

from ..base.exceptions import InputTypeError
from ..engine.noise_allocation import paired_noise_stddevs
from ..engine.random import RngKey, fold_in
from ..engine.types import ClippedPytree, NoisedPytree, NoiseState, SecondMomentClippingOutput, SecondMomentNoiseOutput


@dataclass(frozen=True)
class PairedMFNoiseState(NoiseState):
    _first: Any
    _second: Any
    _step_counter: int
    _rng_key: RngKey


def make_second_moment_mf_noise(grad_template, strategy, second_strategy, *, n_steps, min_sep, max_participations,
                                noise_multiplier, key, compute_dtype=torch.float32, backend="auto"):
    from .noise import SECOND_MOMENT_FIRST_FOLD, SECOND_MOMENT_SECOND_FOLD, mf_gaussian_noise

    kw = dict(n_steps=n_steps, min_sep=min_sep, max_participations=max_participations, compute_dtype=compute_dtype,
              backend=backend)
    s1 = strategy.sensitivity(n_steps=n_steps, min_sep=min_sep, max_participations=max_participations)
    s2 = second_strategy.sensitivity(n_steps=n_steps, min_sep=min_sep, max_participations=max_participations)
    # unit-multiplier raw streams; the joint allocation decides each stream's scale per step
    f1, st1 = mf_gaussian_noise(grad_template, strategy, noise_multiplier=1.0, key=fold_in(key, SECOND_MOMENT_FIRST_FOLD), **kw)
    f2, st2 = mf_gaussian_noise(grad_template, second_strategy, noise_multiplier=1.0,
                                key=fold_in(key, SECOND_MOMENT_SECOND_FOLD), **kw)

    def noise_fn(inp, st: PairedMFNoiseState):
        if not isinstance(inp, SecondMomentClippingOutput):
            raise InputTypeError("this mechanism was built with a second-moment strategy and expects "
                                 "SecondMomentClippingOutput inputs")
        a, b = inp.grads, inp.squared_grads
        d1, d2 = a.max_norm * s1, b.max_norm * s2
        sig1, sig2 = paired_noise_stddevs(noise_multiplier, first=d1, second=d2)
        # feed each raw stream a ClippedPytree whose max_norm makes nm=1 produce the allotted sigma
        n1, st1n = f1(ClippedPytree(a.pytree, sig1), replace(st._first, _first_max_norm=None))
        n2, st2n = f2(ClippedPytree(b.pytree, sig2), replace(st._second, _first_max_norm=None))
        out = SecondMomentNoiseOutput(NoisedPytree(n1.pytree, a.max_norm, n1.noise_stddev),
                                      NoisedPytree(n2.pytree, b.max_norm, n2.noise_stddev))
        return out, PairedMFNoiseState(st1n, st2n, st._step_counter + 1, st._rng_key)

    return noise_fn, PairedMFNoiseState(st1, st2, 0, key)
