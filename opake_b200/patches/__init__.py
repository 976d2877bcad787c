"""Model and runtime patches (counterpart of ``opake.patches``, packages/opake-patches/src/opake/api/patches/
__init__.py:20-164).

``apply_runtime_patches`` registers process-wide hooks (the fused clip-and-sum backend of the generic clipping path).
``apply_model_patches`` rewires one Hugging Face model so that it is legal and fast under ``vmap(grad)``: dropout and
KV cache off, vmap-safe attention, RMSNorm / gated-MLP forwards on the fused kernels, LoRA layers on the fused LoRA
function, optionally the LM head + loss on the fused linear cross-entropy. Families that the native runtime supports
can instead be lowered completely with ``to_native``.
"""
from __future__ import annotations

import types

from ..engine.clipping.kernel_backend import get_fused_clip_backend, register_fused_clip_backend
from . import kernels, peft, torch_checkpoint
from .peft import apply_peft_model_patches
from .transformers.registry import FAMILIES, FamilySpec, family_of

__all__ = ["apply_model_patches", "apply_runtime_patches", "apply_peft_model_patches", "apply_transformers_model_patches",
           "is_runtime_patched", "to_native", "FAMILIES", "family_of", "kernels"]

_RUNTIME = {"patched": False}


def is_runtime_patched() -> bool:
    return _RUNTIME["patched"]


def apply_runtime_patches(*, performance: bool = True, compat: bool = True, **kw) -> dict:
    """Idempotent process-wide patches; returns what this call changed.

    ``performance``: registers the CUDA multi-tensor clip-and-sum as the fused clipping backend. ``compat`` turns on,
    each overridable by keyword: ``vmap_masking`` (mask builders legal under ``vmap(grad)``), ``empty_batches``
    (collators that survive an empty Poisson batch), ``vmap_grouped_mm`` (grouped expert GEMM gate),
    ``vmap_checkpointing`` (layer checkpointing under functorch: see ``patches.torch_checkpoint``)."""
    report = {"fused_clip_backend": False, "masking": 0, "collators": 0, "grouped_mm": False}
    if performance and get_fused_clip_backend() is None:
        from ..ops import clip_sum
        register_fused_clip_backend(clip_sum)
        report["fused_clip_backend"] = True
    from .transformers import runtime as R
    if kw.get("vmap_masking", compat):
        report["masking"] = R.apply_masking_patches()
    if kw.get("empty_batches", compat):
        report["collators"] = R.apply_collator_patches()
    if kw.get("vmap_grouped_mm", compat):
        report["grouped_mm"] = R.apply_grouped_mm_patches()
    _RUNTIME["patched"] = True
    return report


def apply_transformers_model_patches(model, *, performance: bool = True, compat: bool = True, kernels: bool | None = None,
                                     fused_linear_cross_entropy: bool | None = None, **cfg) -> dict:
    """Patches a Hugging Face decoder in place; returns a report ``{what: count}``.

    Umbrella flags and the per-concern keywords they default: ``compat`` -> ``dropout``, ``batchify``,
    ``eager_attention`` (vmap-safe attention interface); ``performance`` -> ``kv_cache``, ``fused_linear_cross_entropy``
    (conditional ``loss_only`` forward); ``kernels`` (defaults to ``performance``) -> ``rms_norm``, ``activation``,
    ``rope``, ``cross_entropy`` (the model's ``loss_function``)."""
    from .transformers import components as C
    from .transformers.family import family_name, get_family_apply_fn

    user_apply = get_family_apply_fn(family_name(model))
    if user_apply is not None:          # a family registered with an apply function handles itself
        out = user_apply(model, performance=performance, compat=compat, kernels=kernels,
                         fused_linear_cross_entropy=performance if fused_linear_cross_entropy is None else fused_linear_cross_entropy,
                         **cfg)
        return out if isinstance(out, dict) else {"family": family_name(model)}
    spec = family_of(model)
    kernels = performance if kernels is None else kernels
    report = {"family": spec.model_type if spec else None, "norms": 0, "mlps": 0, "dropouts": 0, "attention": None, "kv_cache": 0,
              "batchify": 0, "rope": 0, "loss_function": 0, "fused_linear_cross_entropy": False}
    root_cls = type(model)
    # forward wrappers nest: the fused-loss branch innermost, the batch-dimension shim outermost (each wrapper copies the
    # marks of what it wraps, so a second application sees all of them on the outermost function)
    fused = performance if fused_linear_cross_entropy is None else fused_linear_cross_entropy
    if fused:
        report["fused_linear_cross_entropy"] = C.apply_fused_linear_ce_patch(model)
    if cfg.get("dropout", compat):
        report["dropouts"] = C.disable_dropout(model)
    if cfg.get("kv_cache", performance):
        C.disable_kv_cache(model)
        report["kv_cache"] = C.apply_kv_cache_patch(root_cls, model) if hasattr(model, "config") else 0
    if cfg.get("batchify", compat) and hasattr(model, "config"):
        report["batchify"] = C.apply_batchify_patch(root_cls, model)
    if compat:
        conf = getattr(model, "config", None)
        if conf is not None and hasattr(conf, "_attn_implementation"):
            try:
                from transformers import AttentionInterface
                name = "opake_eager" if cfg.get("eager_attention") or (spec and spec.softcap) else "opake_sdpa"
                AttentionInterface.register("opake_sdpa", C.vmap_sdpa_attention_forward)
                AttentionInterface.register("opake_eager", C.eager_attention_forward)
                conf._attn_implementation = name
                report["attention"] = name
            except Exception:
                report["attention"] = "stock"
    if kernels and spec is not None:
        for m in model.modules():
            cname = type(m).__name__
            if cfg.get("rms_norm", True) and spec.norm_suffixes and cname.endswith(spec.norm_suffixes) and hasattr(m, "weight") \
                    and not hasattr(m, "bias") and not hasattr(m, "_opake_patched"):
                m._opake_offset, m._opake_patched = spec.norm_offset, True
                m.forward = types.MethodType(C.patched_rms_norm_forward, m)
                report["norms"] += 1
            elif cfg.get("activation", True) and spec.mlp_suffixes and cname.endswith(spec.mlp_suffixes) and not hasattr(m, "_opake_patched"):
                if all(hasattr(m, a) for a in ("gate_proj", "up_proj", "down_proj")):
                    fwd = C.patched_gated_mlp_forward
                elif spec.fused_gate_up and all(hasattr(m, a) for a in ("gate_up_proj", "down_proj")):
                    fwd = C.patched_fused_gate_up_mlp_forward
                else:
                    continue
                m._opake_act, m._opake_patched = spec.act, True
                m.forward = types.MethodType(fwd, m)
                report["mlps"] += 1
        if cfg.get("rope", True) and spec.rope:
            report["rope"] = C.apply_rope_patch(model)
    if kernels and cfg.get("cross_entropy", True) and hasattr(model, "loss_function") and hasattr(model, "lm_head"):
        report["loss_function"] = C.apply_causal_lm_loss_function_patch(model, root_cls)
    return report


def apply_model_patches(model, *, performance: bool = True, compat: bool = True, peft: bool = True,
                        fused_linear_cross_entropy: bool | None = None, kernels: bool = True, **kwargs) -> dict:
    apply_runtime_patches(performance=performance, compat=compat)
    report = {}
    if hasattr(model, "config") and not hasattr(model, "flat"):
        report = apply_transformers_model_patches(model, performance=performance, compat=compat, kernels=kernels,
                                                  fused_linear_cross_entropy=fused_linear_cross_entropy, **kwargs)
    if peft:
        report["lora_layers"] = apply_peft_model_patches(model)
    return report


def to_native(model, dtype=None, device=None):
    """Lowers a supported Hugging Face decoder to ``NativeCausalLM`` (flat parameters, sm_100a runtime)."""
    import torch
    from ..base.exceptions import ConfigurationError
    from ..models.native import NativeCausalLM
    spec = family_of(model)
    if spec is None or not spec.native:
        raise ConfigurationError(f"model family {getattr(getattr(model, 'config', None), 'model_type', None)!r} has no native "
                                 "lowering; use apply_model_patches for the generic path")
    return NativeCausalLM.from_hf(model, dtype=dtype or torch.float32, device=device)
