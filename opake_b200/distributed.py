"""Public namespace ``opake_b200.distributed`` (the ``opake.distributed`` façade of the reference, packages/opake-engine/src/opake/distributed/__init__.py): re-exports
``opake_b200.engine.distributed``."""
from .engine.distributed import *  # noqa: F401,F403
from .engine.distributed import __all__  # noqa: F401
