"""``torchopt.base`` stand-in: the functional optimizer protocol (``init`` / ``update`` pairs) and ``chain``."""
from __future__ import annotations

from typing import Any, Callable, NamedTuple


class EmptyState(NamedTuple):
    """State of a transformation that keeps none."""


class GradientTransformation(NamedTuple):
    """``init(params) -> state`` and ``update(updates, state, *, params=None, inplace=True) -> (updates, state)``."""

    init: Callable[..., Any]
    update: Callable[..., Any]

    def chain(self, next_: "GradientTransformation") -> "GradientTransformation":
        return chain(self, next_)


class ChainedGradientTransformation(GradientTransformation):
    """A sequence of transformations applied one after the other; its state is the tuple of their states."""

    transformations: tuple

    def __new__(cls, *transformations: GradientTransformation):
        flat: list[GradientTransformation] = []
        for t in transformations:
            if isinstance(t, ChainedGradientTransformation):
                flat.extend(t.transformations)
            elif isinstance(t, IdentityGradientTransformation):
                continue
            else:
                flat.append(t)
        flat_t = tuple(flat)

        def init_fn(params):
            return tuple(t.init(params) for t in flat_t)

        def update_fn(updates, state, *, params=None, inplace=True):
            if len(flat_t) != len(state):
                raise ValueError("the number of updates and states has to be the same in chain")
            new_state = []
            for s, t in zip(state, flat_t):
                updates, ns = t.update(updates, s, params=params, inplace=inplace)
                new_state.append(ns)
            return updates, tuple(new_state)

        inst = super().__new__(cls, init_fn, update_fn)
        inst.transformations = flat_t
        return inst


class IdentityGradientTransformation(GradientTransformation):
    def __new__(cls):
        return super().__new__(cls, lambda params: EmptyState(), lambda updates, state, *, params=None, inplace=True: (updates, state))


def identity() -> GradientTransformation:
    return IdentityGradientTransformation()


def chain(*transformations: GradientTransformation) -> GradientTransformation:
    if len(transformations) == 0:
        return identity()
    if len(transformations) == 1:
        return transformations[0]
    return ChainedGradientTransformation(*transformations)
