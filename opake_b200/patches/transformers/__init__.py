"""Hugging Face model patches (packages/opake-patches/src/opake/patches/transformers/__init__.py): the dispatcher, the
family registry and the factories with which a downstream architecture registers itself."""
from .family import (family_name, get_family_apply_fn, make_apply_family_patches, make_apply_model_patches,
                     register_activation_kind, register_family, register_fused_add_rms_kind, register_moe_kind,
                     register_rms_norm_kind, supported_families)
from .registry import FAMILIES, FamilySpec, family_of


def apply_transformers_model_patches(model, **kwargs):
    from .. import apply_transformers_model_patches as _apply

    return _apply(model, **kwargs)


__all__ = ["apply_transformers_model_patches", "family_name", "make_apply_family_patches", "make_apply_model_patches",
           "register_activation_kind", "register_family", "register_fused_add_rms_kind", "register_moe_kind",
           "register_rms_norm_kind", "supported_families", "get_family_apply_fn", "FAMILIES", "FamilySpec", "family_of"]
