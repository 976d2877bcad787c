"""Public namespace ``opake_b200.functional`` (the ``opake.functional`` façade of the reference, packages/opake-engine/src/opake/functional/__init__.py): re-exports
``opake_b200.engine.functional``."""
from .engine.functional import *  # noqa: F401,F403
from .engine.functional import __all__  # noqa: F401
