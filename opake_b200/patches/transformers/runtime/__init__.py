"""Process-wide Hugging Face patches (packages/opake-patches/src/opake/api/patches/transformers/runtime/): collators
that survive empty Poisson batches, a vmap-safe grouped-GEMM gate for stacked experts, vmap-safe mask builders."""
from .collator import apply_collator_patches
from .masking import apply_masking_patches
from .moe import apply_grouped_mm_patches

__all__ = ["apply_collator_patches", "apply_grouped_mm_patches", "apply_masking_patches"]
