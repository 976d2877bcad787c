"""Public namespace ``opake_b200.scheduling`` (the ``opake.scheduling`` façade of the reference, packages/opake-engine/src/opake/scheduling/__init__.py): re-exports
``opake_b200.engine.scheduling``."""
from .engine.scheduling import *  # noqa: F401,F403
from .engine.scheduling import __all__  # noqa: F401
