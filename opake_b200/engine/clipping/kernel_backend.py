"""Hook through which the CUDA clip-sum kernels plug into the generic clipping path
(reference: packages/opake-engine/src/opake/api/engine/clipping/_kernel_backend.py:9-17)."""
from __future__ import annotations

_BACKEND = None


def register_fused_clip_backend(fn) -> None:
    global _BACKEND
    _BACKEND = fn


def get_fused_clip_backend():
    return _BACKEND
