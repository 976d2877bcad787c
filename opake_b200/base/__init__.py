"""Layer 1: exception taxonomy and the serialization registry (no third-party dependencies)."""
from . import exceptions, serialization  # noqa: F401
