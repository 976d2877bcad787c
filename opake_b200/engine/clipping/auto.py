"""AUTO-S normalisation clipping: every example is rescaled by ``R / (norm + gamma)`` (Bu et al.).

Same factory shape as fixed clipping (packages/opake-engine/src/opake/api/engine/clipping/_auto.py:112-367); the
output sensitivity is ``R / normalize_by``.
"""
from __future__ import annotations

from dataclasses import dataclass

from ...base.exceptions import ConfigurationError
from ..types import ClipState
from .core import _BuiltinScale, _identity, clipped_fun, clipped_grad


@dataclass(frozen=True)
class AutoClipState(ClipState):
    """Marker state of AUTO-S clipping."""


def _check(R, gamma):
    if not (R > 0):
        raise ConfigurationError(f"R must be positive, got {R}")
    if not (gamma > 0):
        raise ConfigurationError(f"gamma must be positive, got {gamma}")


def _restate(fn):
    def wrapped(*args, state, **kwargs):
        out, _ = fn(*args, state=_INNER, **kwargs)
        return out, state

    return wrapped


from .core import FixedClipState  # noqa: E402

_INNER = FixedClipState()


def auto_clipped_fun(fun, has_aux=False, *, batch_argnums=0, R: float = 1.0, gamma: float = 0.01, normalize_by=1.0,
                     return_aux=False, return_stats=False, microbatch_size=None, dtype=None, second_moment=False,
                     _chunk_compiler=None):
    _check(R, gamma)
    fn, _ = clipped_fun(fun, has_aux, batch_argnums=batch_argnums, clipping_norm=R, normalize_by=normalize_by,
                        return_aux=return_aux, return_stats=return_stats, second_moment=second_moment,
                        microbatch_size=microbatch_size, dtype=dtype, _builtin_scale=_BuiltinScale("auto", gamma),
                        _chunk_compiler=_chunk_compiler)
    return _restate(fn), AutoClipState()


def auto_clipped_grad(loss_fn, argnums=0, has_aux=False, *, R: float = 1.0, gamma: float = 0.01, normalize_by=1.0,
                      batch_argnums=1, return_aux=False, return_stats=False, pre_clipping_transform=_identity,
                      microbatch_size=None, dtype=None, second_moment=False, _chunk_compiler=None):
    _check(R, gamma)
    fn, _ = clipped_grad(loss_fn, argnums, has_aux, clipping_norm=R, normalize_by=normalize_by,
                         batch_argnums=batch_argnums, return_aux=return_aux, return_stats=return_stats,
                         second_moment=second_moment, pre_clipping_transform=pre_clipping_transform,
                         microbatch_size=microbatch_size, dtype=dtype, _builtin_scale=_BuiltinScale("auto", gamma),
                         _chunk_compiler=_chunk_compiler)
    return _restate(fn), AutoClipState()


__all__ = ["AutoClipState", "auto_clipped_fun", "auto_clipped_grad"]
