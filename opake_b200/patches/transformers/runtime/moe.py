"""vmap-safe gate for the grouped expert GEMM of Hugging Face v5 (packages/opake-patches/src/opake/api/patches/
transformers/runtime/moe.py). ``transformers.integrations.moe._can_use_grouped_mm`` reads ``weight.data_ptr()`` for an
alignment check; under ``vmap(grad)`` the tensors are batched views without storage and the read raises. Inside a
functorch transform the gate therefore answers from the availability of the grouped kernel alone."""
from __future__ import annotations

import torch

from ....engine.functional import under_differentiating_transform

__all__ = ["apply_grouped_mm_patches"]


def _inside_functorch() -> bool:
    try:
        from torch._C._functorch import maybe_current_level     # type: ignore[attr-defined]

        return maybe_current_level() is not None
    except Exception:
        return under_differentiating_transform()


def apply_grouped_mm_patches(*, vmap_grouped_mm: bool = True) -> bool:
    if not vmap_grouped_mm:
        return False
    try:
        import transformers.integrations.moe as moe
    except ImportError:
        return False
    orig = getattr(moe, "_can_use_grouped_mm", None)
    if orig is None or getattr(orig, "_opake_vmap_safe", False):
        return False

    def can_use_grouped_mm(input, weight, offs):
        try:
            return orig(input, weight, offs)
        except RuntimeError:
            if _inside_functorch():
                return hasattr(torch.nn.functional, "grouped_mm") or hasattr(torch, "_grouped_mm")
            raise

    can_use_grouped_mm._opake_vmap_safe = True
    can_use_grouped_mm._original = orig
    moe._can_use_grouped_mm = can_use_grouped_mm
    return True
