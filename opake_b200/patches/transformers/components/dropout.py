"""Dropout off for DP training (packages/opake-patches/src/opake/api/patches/transformers/components/dropout.py).

Per-example clipping plus noise is the regulariser, and module dropout has no per-example randomness under ``vmap``
(the fused dropout of SDPA refuses batched inputs outright). Three places carry a rate: ``nn.Dropout`` modules, float
attributes that forwards read directly (``self.attention_dropout`` handed to SDPA), and the config."""
from __future__ import annotations

import torch.nn as nn

__all__ = ["disable_dropout", "DROPOUT_ATTRS"]

DROPOUT_ATTRS = ("attention_dropout", "dropout", "hidden_dropout", "ffn_dropout", "attn_pdrop", "resid_pdrop", "embd_pdrop",
                 "attention_probs_dropout_prob", "hidden_dropout_prob", "classifier_dropout", "summary_first_dropout")


def _zero_float_attrs(obj) -> int:
    n = 0
    for name in DROPOUT_ATTRS:
        v = getattr(obj, name, None)
        if isinstance(v, float) and v != 0.0:          # bool is an int subclass but never a rate: floats only
            try:
                setattr(obj, name, 0.0)
                n += 1
            except AttributeError:                      # read-only property
                pass
    return n


def disable_dropout(model) -> int:
    """Zeroes every dropout source of ``model``; returns how many were non-zero."""
    modules = getattr(model, "modules", None)
    if not callable(modules):
        return 0
    n = 0
    for m in modules():
        if isinstance(m, nn.modules.dropout._DropoutNd):
            if m.p:
                m.p, n = 0.0, n + 1
        else:
            n += _zero_float_attrs(m)
    cfg = getattr(model, "config", None)
    if cfg is not None:
        n += _zero_float_attrs(cfg)
    return n
