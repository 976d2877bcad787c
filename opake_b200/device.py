"""Public namespace ``opake_b200.device`` (the ``opake.device`` façade of the reference, packages/opake-engine/src/opake/device/__init__.py): re-exports
``opake_b200.engine.device``."""
from .engine.device import *  # noqa: F401,F403
from .engine.device import __all__  # noqa: F401
