"""Batch-dimension shim for model forwards (packages/opake-patches/src/opake/api/patches/transformers/components/
batchify.py). Under ``vmap(grad)`` one example arrives without its batch axis (``input_ids`` of shape ``[T]``); Hugging
Face forwards assume ``[B, T]``. The wrapper adds the axis on entry and strips it from the outputs; already batched
calls pass through."""
from __future__ import annotations

import types

from ....engine.functional import with_batch_dim

__all__ = ["batchify_forward", "apply_batchify_patch"]

_MARK = "_opake_batchified"
_KWARG_NDIM = {"input_ids": 2, "attention_mask": 2, "labels": 2, "position_ids": 2, "token_type_ids": 2, "inputs_embeds": 3}


def batchify_forward(forward_fn):
    if getattr(forward_fn, _MARK, False):
        return forward_fn
    wrapped = with_batch_dim(forward_fn, batch_argnums=(1,), batch_kwargs=_KWARG_NDIM, min_ndim=2)    # 0 is ``self``
    setattr(wrapped, _MARK, True)
    return wrapped


def apply_batchify_patch(target_cls: type | None, model=None) -> int:
    if target_cls is None:
        return 0
    n = 0
    fwd = getattr(target_cls, "forward", None)
    if fwd is not None and not getattr(fwd, _MARK, False):
        target_cls.forward = batchify_forward(fwd)
        n += 1
    if model is not None:
        for m in model.modules():
            if type(m) is target_cls and "forward" in m.__dict__:
                inst = m.__dict__["forward"]
                unbound = getattr(inst, "__func__", inst)
                if not getattr(unbound, _MARK, False):
                    m.forward = types.MethodType(batchify_forward(unbound), m)
                    n += 1
    return n
