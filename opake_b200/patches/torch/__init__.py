"""Layer checkpointing under functorch transforms (packages/opake-patches/src/opake/patches/torch/__init__.py).

``torch.utils.checkpoint`` refuses to run inside ``vmap(grad)``. ``apply_checkpoint_patch`` routes the Hugging Face
gradient-checkpointing hook (``GradientCheckpointingLayer`` calls ``self._gradient_checkpointing_func``) and
``torch.utils.checkpoint.checkpoint`` itself, WHEN CALLED INSIDE A TRANSFORM, to the functional recomputation of
``patches.torch_checkpoint``; outside a transform the stock function runs."""
from __future__ import annotations

import functools

from ..torch_checkpoint import (apply_gradient_checkpointing, checkpoint_under_vmap, hf_checkpoint_under_transforms,
                                offload_activations)

__all__ = ["apply_checkpoint_patch", "is_checkpoint_patched", "checkpoint_under_vmap", "hf_checkpoint_under_transforms",
           "apply_gradient_checkpointing", "offload_activations"]

_STATE = {"patched": False, "original": None}


def _inside_transform() -> bool:
    try:
        from torch._C._functorch import maybe_current_level     # type: ignore[attr-defined]

        return maybe_current_level() is not None
    except Exception:
        return False


def apply_checkpoint_patch(*, vmap_checkpointing: bool = True) -> bool:
    """Idempotent; returns whether this call installed the patch."""
    if not vmap_checkpointing or _STATE["patched"]:
        return False
    import torch.utils.checkpoint as tuc

    original = tuc.checkpoint

    @functools.wraps(original)
    def checkpoint(function, *args, **kwargs):
        if _inside_transform():
            for k in ("use_reentrant", "preserve_rng_state", "determinism_check", "context_fn", "debug"):
                kwargs.pop(k, None)
            import torch
            import torch.nn as nn

            bound = getattr(getattr(function, "func", function), "__self__", None)
            if isinstance(bound, nn.Module) and not kwargs:
                return hf_checkpoint_under_transforms(function, *args)
            if args and not kwargs and all(isinstance(a, torch.Tensor) and a.is_floating_point() for a in args):
                return checkpoint_under_vmap(function, *args)
            return function(*args, **kwargs)          # nothing to recompute safely: run it plainly (correct, not lean)
        return original(function, *args, **kwargs)

    checkpoint._opake_vmap_safe = True
    tuc.checkpoint = checkpoint
    _STATE.update(patched=True, original=original)
    return True


def is_checkpoint_patched() -> bool:
    return bool(_STATE["patched"])
