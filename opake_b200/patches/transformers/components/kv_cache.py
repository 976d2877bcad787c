"""KV cache off while training (packages/opake-patches/src/opake/api/patches/transformers/components/kv_cache.py).

Hugging Face decoders default to ``use_cache=True`` and build a ``DynamicCache`` in every forward pass; in training it
is never read, and under ``vmap`` the cache objects keep batched tensors alive through reference cycles. The wrapper
forces ``use_cache=False`` only when gradients are enabled, the module is in training mode and no cache with content
was passed, so generation (which hands over an empty cache and fills it) keeps working."""
from __future__ import annotations

import functools
import types

import torch

__all__ = ["disable_kv_cache_in_training", "apply_kv_cache_patch", "disable_kv_cache"]

_MARK = "_opake_cache_disabled"


def _has_cached_data(past) -> bool:
    if past is None:
        return False
    if hasattr(past, "get_seq_length"):
        try:
            return past.get_seq_length() > 0
        except Exception:
            return False
    try:
        return len(past) > 0
    except TypeError:
        return False


def disable_kv_cache_in_training(forward_fn):
    if getattr(forward_fn, _MARK, False):
        return forward_fn

    @functools.wraps(forward_fn)
    def wrapper(*args, **kwargs):
        model = args[0] if args else None
        if torch.is_grad_enabled() and getattr(model, "training", False) and not _has_cached_data(kwargs.get("past_key_values")):
            kwargs["use_cache"] = False
        return forward_fn(*args, **kwargs)

    setattr(wrapper, _MARK, True)
    return wrapper


def apply_kv_cache_patch(target_cls: type | None, model=None) -> int:
    """Wraps ``target_cls.forward`` (every instance) and instance-level forwards of ``model``'s modules of that class
    that were overridden before. Returns the number of wrappers installed."""
    if target_cls is None:
        return 0
    n = 0
    fwd = target_cls.__dict__.get("forward", getattr(target_cls, "forward", None))
    if fwd is not None and not getattr(fwd, _MARK, False):
        target_cls.forward = disable_kv_cache_in_training(fwd)
        n += 1
    if model is not None:
        for m in model.modules():
            if type(m) is target_cls and "forward" in m.__dict__:
                inst = m.__dict__["forward"]
                unbound = getattr(inst, "__func__", inst)
                if not getattr(unbound, _MARK, False):
                    m.forward = types.MethodType(disable_kv_cache_in_training(unbound), m)
                    n += 1
    return n


def disable_kv_cache(model) -> None:
    """Config-level switch (kept for models whose forward cannot be wrapped)."""
    cfg = getattr(model, "config", None)
    if cfg is not None and getattr(cfg, "use_cache", False):
        cfg.use_cache = False
