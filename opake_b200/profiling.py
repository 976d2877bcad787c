"""Public namespace ``opake_b200.profiling`` (the ``opake.profiling`` façade of the reference, packages/opake-engine/src/opake/profiling/__init__.py): re-exports
``opake_b200.engine.profiling``."""
from .engine.profiling import *  # noqa: F401,F403
from .engine.profiling import __all__  # noqa: F401
