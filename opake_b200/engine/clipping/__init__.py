from .core import (ClippedFunAux, ClippedGradAux, ClippingStats, FixedClipState, clipped_fun, clipped_grad)  # noqa: F401
