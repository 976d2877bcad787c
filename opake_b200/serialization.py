"""Public namespace ``opake_b200.serialization`` (the ``opake.serialization`` façade of the reference, packages/opake-base/src/opake/serialization/__init__.py): re-exports
``opake_b200.base.serialization``."""
from .base.serialization import *  # noqa: F401,F403
from .base.serialization import __all__  # noqa: F401
