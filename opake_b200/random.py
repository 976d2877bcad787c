"""Public namespace ``opake_b200.random`` (the ``opake.random`` façade of the reference, packages/opake-engine/src/opake/random/__init__.py): re-exports
``opake_b200.engine.random``."""
from .engine.random import *  # noqa: F401,F403
from .engine.random import __all__  # noqa: F401
