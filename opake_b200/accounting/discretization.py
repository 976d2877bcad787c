"""Process-global discretization settings of the accountant with per-call overrides.

Defaults and override names follow packages/opake-accounting/src/opake/api/accounting/core/discretization.py:17-272:
grid 1e-4, log mass truncation -50, max grid 10 000 000, tail truncation 1e-15, seed 42, max convolution grid 32 768,
Monte-Carlo resolution 1e-5 and failure probability 1e-6.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, replace

from ..base.exceptions import ConfigurationError
from ._native import native


@dataclass(frozen=True)
class _Settings:
    discretization: float = 1e-4
    log_x_mass_truncation_bound: float = -50.0
    max_grid_size: int = 10_000_000
    tail_mass_truncation: float = 1e-15
    seed: int = 42
    max_conv_grid: int = 32_768
    mc_resolution: float = 1e-5
    mc_failure_probability: float = 1e-6


_LOCK = threading.RLock()
_CURRENT = _Settings()
OVERRIDE_NAMES = ("discretization", "log_x_mass_truncation_bound", "max_grid_size", "max_conv_grid", "seed",
                  "mc_resolution", "mc_failure_probability")


def _validated(s: _Settings) -> _Settings:
    if not s.discretization > 0:
        raise ConfigurationError(f"discretization must be > 0, got {s.discretization}")
    if not s.log_x_mass_truncation_bound < 0:
        raise ConfigurationError("log_x_mass_truncation_bound must be negative")
    if s.max_grid_size < 2 or s.max_conv_grid < 2:
        raise ConfigurationError("grid sizes must be >= 2")
    if not 0 < s.mc_resolution < 1 or not 0 < s.mc_failure_probability < 1:
        raise ConfigurationError("mc_resolution and mc_failure_probability must be in (0, 1)")
    return s


def set_discretization(**kwargs) -> None:
    """Change the global defaults (keyword names as in :data:`OVERRIDE_NAMES` plus ``tail_mass_truncation``)."""
    global _CURRENT
    with _LOCK:
        _CURRENT = _validated(replace(_CURRENT, **{k: v for k, v in kwargs.items() if v is not None}))


def reset_discretization() -> None:
    global _CURRENT
    with _LOCK:
        _CURRENT = _Settings()


def get_discretization(**overrides):
    """Native ``DiscretizationConfig`` for the global settings with the given non-``None`` overrides applied."""
    with _LOCK:
        s = _CURRENT
    s = _validated(replace(s, **{k: v for k, v in overrides.items() if v is not None}))
    return native().DiscretizationConfig(s.discretization, s.log_x_mass_truncation_bound, s.max_grid_size,
                                         s.tail_mass_truncation, s.seed, s.max_conv_grid, s.mc_resolution,
                                         s.mc_failure_probability)


__all__ = ["set_discretization", "get_discretization", "reset_discretization", "OVERRIDE_NAMES"]
