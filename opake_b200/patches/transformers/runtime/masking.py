"""vmap-safe attention-mask builders (packages/opake-patches/src/opake/api/patches/transformers/runtime/
masking.py:253,415,608,626).

The Hugging Face builders decide with data-dependent Python control flow (``padding_mask.all()``, cache lengths read
from tensors), which is illegal inside ``vmap(grad)``. Inside a functorch transform the replacements below build the
mask from iota comparisons only: causal (and sliding-window) structure, padding, and user mask hooks
(``or_mask_function`` / ``and_mask_function``) evaluated on broadcastable index tensors. Outside a transform, and
whenever a cache with content is passed (generation), the original builder runs, so stock behaviour is untouched.

``transformers`` modules bind the builders by name at import time (``from ...masking_utils import create_causal_mask``),
so the patch rebinds the name in ``masking_utils`` AND in every already imported ``transformers.models.*`` module."""
from __future__ import annotations

import sys

import torch

__all__ = ["apply_masking_patches", "vmap_create_causal_mask", "vmap_create_sliding_window_causal_mask",
           "vmap_safe_ignore_causal_mask_sdpa", "build_mask"]

_ORIGINALS: dict[str, object] = {}
_BOOL_BACKENDS = ("sdpa", "opake_sdpa", "opake_eager", "flex_attention")


def _inside_transform() -> bool:
    try:
        from torch._C._functorch import maybe_current_level     # type: ignore[attr-defined]

        return maybe_current_level() is not None
    except Exception:
        return False


def _cache_has_content(past) -> bool:
    if past is None:
        return False
    try:
        return int(past.get_seq_length()) > 0
    except Exception:
        return False


def build_mask(q_len: int, attention_mask, device, *, window: int | None = None, or_mask_function=None, and_mask_function=None,
               batch_size: int = 1) -> torch.Tensor:
    """Boolean ``[B, 1, q_len, q_len]`` mask (True = attend) of a cache-free forward pass."""
    qi = torch.arange(q_len, device=device).view(1, 1, -1, 1)
    ki = torch.arange(q_len, device=device).view(1, 1, 1, -1)
    allowed = ki <= qi
    if window is not None:
        allowed = allowed & (ki > qi - int(window))
    if or_mask_function is not None or and_mask_function is not None:
        b = torch.arange(batch_size, device=device).view(-1, 1, 1, 1)
        h = torch.zeros(1, dtype=torch.long, device=device)

        def hook(fn):
            r = fn(b, h, qi, ki)
            return r.to(device=device, dtype=torch.bool) if isinstance(r, torch.Tensor) else torch.full((), bool(r), device=device)

        if or_mask_function is not None:
            allowed = allowed | hook(or_mask_function)
        if and_mask_function is not None:
            allowed = allowed & hook(and_mask_function)
    if attention_mask is not None:
        allowed = allowed & attention_mask[..., None, None, :q_len].to(torch.bool)
    return allowed.expand(batch_size if attention_mask is None else attention_mask.shape[0], 1, q_len, q_len)


def _finish(mask: torch.Tensor, config, dtype: torch.dtype):
    impl = getattr(config, "_attn_implementation", None)
    if impl in _BOOL_BACKENDS:
        return mask
    return torch.zeros((), dtype=dtype, device=mask.device).masked_fill(~mask, torch.finfo(dtype).min)   # additive (eager)


def _vmap_builder(name: str, windowed: bool):
    def builder(config, inputs_embeds, attention_mask, cache_position=None, *, past_key_values=None, position_ids=None,
                or_mask_function=None, and_mask_function=None, **extra):
        if not _inside_transform() or _cache_has_content(past_key_values):
            return _ORIGINALS[name](config, inputs_embeds, attention_mask, cache_position, past_key_values=past_key_values,
                                    position_ids=position_ids, or_mask_function=or_mask_function,
                                    and_mask_function=and_mask_function, **extra)
        q_len = inputs_embeds.shape[-2]
        window = None
        if windowed:
            cfg = config.get_text_config() if hasattr(config, "get_text_config") else config
            window = getattr(cfg, "sliding_window", None)
            if window is not None and window >= q_len:
                window = None
        impl = getattr(config, "_attn_implementation", None)
        if attention_mask is None and or_mask_function is None and and_mask_function is None and impl in ("opake_sdpa", "opake_eager"):
            return None         # this package's attention functions rebuild causal / windowed structure from the shapes
        if attention_mask is not None and attention_mask.dim() == 4:
            return attention_mask          # the caller already built a mask
        mask = build_mask(q_len, attention_mask, inputs_embeds.device, window=window, or_mask_function=or_mask_function,
                          and_mask_function=and_mask_function, batch_size=inputs_embeds.shape[0] if inputs_embeds.dim() == 3 else 1)
        return _finish(mask, config, inputs_embeds.dtype)

    builder.__name__ = "vmap_" + name
    builder._opake_vmap_safe = True
    return builder


vmap_create_causal_mask = _vmap_builder("create_causal_mask", windowed=False)
vmap_create_sliding_window_causal_mask = _vmap_builder("create_sliding_window_causal_mask", windowed=True)


def vmap_safe_ignore_causal_mask_sdpa(*args, **kwargs) -> bool:
    """The original asks ``padding_mask.all()``. With a padding mask the answer here is "do not ignore" (the mask is
    needed for the padding anyway); without one the remaining checks are on Python ints and the original decides.
    Arguments are forwarded unread: their order changed between library releases."""
    padding_mask = args[0] if args else kwargs.get("padding_mask")
    if padding_mask is not None:
        return False
    return _ORIGINALS["_ignore_causal_mask_sdpa"](*args, **kwargs)


vmap_safe_ignore_causal_mask_sdpa._opake_vmap_safe = True


def apply_masking_patches(*, vmap_masking: bool = True) -> int:
    """Idempotent; returns the number of names rebound by this call."""
    if not vmap_masking:
        return 0
    try:
        import transformers.masking_utils as mu
    except ImportError:
        return 0
    table = {"create_causal_mask": vmap_create_causal_mask,
             "create_sliding_window_causal_mask": vmap_create_sliding_window_causal_mask,
             "_ignore_causal_mask_sdpa": vmap_safe_ignore_causal_mask_sdpa}
    n = 0
    for name, new in table.items():
        cur = getattr(mu, name, None)
        if cur is None or getattr(cur, "_opake_vmap_safe", False):
            continue
        _ORIGINALS[name] = cur
        setattr(mu, name, new)
        n += 1
    # names already bound in imported modeling modules
    for mod_name, mod in list(sys.modules.items()):
        if mod is None or not mod_name.startswith("transformers.models."):
            continue
        for name, new in table.items():
            cur = mod.__dict__.get(name)
            if cur is not None and cur is _ORIGINALS.get(name):
                setattr(mod, name, new)
                n += 1
    return n
