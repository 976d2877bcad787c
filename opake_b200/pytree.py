"""Public namespace ``opake_b200.pytree`` (the ``opake.pytree`` façade of the reference, packages/opake-engine/src/opake/pytree/__init__.py): re-exports
``opake_b200.engine.pytree``."""
from .engine.pytree import *  # noqa: F401,F403
from .engine.pytree import __all__  # noqa: F401
