"""Public namespace ``opake_b200.exceptions`` (the ``opake.exceptions`` façade of the reference, packages/opake-base/src/opake/exceptions/__init__.py): re-exports
``opake_b200.base.exceptions``."""
from .base.exceptions import *  # noqa: F401,F403
from .base.exceptions import __all__  # noqa: F401
