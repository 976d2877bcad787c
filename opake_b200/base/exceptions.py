"""Exception taxonomy of the public API.

Same class names, inheritance and ``raise_`` helper as the reference
(packages/opake-base/src/opake/api/base/exceptions/__init__.py:8-48), so ``except ValueError`` / ``TypeError`` /
``RuntimeError`` handlers written against it keep working.
"""
from __future__ import annotations

from typing import NoReturn

__all__ = ["OpakeError", "ConfigurationError", "InputTypeError", "OperationError", "CalibrationError",
           "PrivacyBudgetError", "CheckpointError"]


class OpakeError(Exception):
    """Root of every failure reported by the framework."""

    @classmethod
    def raise_(cls, message: str, *, cause: BaseException | None = None, suppress_context: bool = False) -> NoReturn:
        err = cls(message)
        if suppress_context:
            raise err from None
        if cause is not None:
            raise err from cause
        raise err


class ConfigurationError(OpakeError, ValueError):
    """Invalid or mutually incompatible settings."""


class InputTypeError(OpakeError, TypeError):
    """An argument has the wrong type."""


class OperationError(OpakeError, RuntimeError):
    """An operation could not finish (device error word set, collective mismatch, ...)."""


class CalibrationError(ConfigurationError):
    """Noise calibration could not bracket or reach the privacy target."""


class PrivacyBudgetError(ConfigurationError):
    """A privacy budget is ill-formed or was used inconsistently."""


class CheckpointError(OperationError):
    """A checkpoint could not be written, read or resumed from."""
