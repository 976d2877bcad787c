"""Debugging utilities of the native runtime (guard-banded buffers)."""
from .canary import CanaryPool, CanaryViolation, DeviceIntegrityError

__all__ = ["CanaryPool", "CanaryViolation", "DeviceIntegrityError"]
