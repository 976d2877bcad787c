"""Public namespace ``opake_b200.types`` (the ``opake.types`` façade of the reference, packages/opake-engine/src/opake/types/__init__.py): re-exports
``opake_b200.engine.types``."""
from .engine.types import *  # noqa: F401,F403
from .engine.types import __all__  # noqa: F401
