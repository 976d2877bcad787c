"""Detached token-level evaluation metrics (packages/opake-alignment/src/opake/api/alignment/metric/_token.py:17-71)."""
from __future__ import annotations

import torch

__all__ = ["entropy_from_logits", "mean_token_accuracy"]


def entropy_from_logits(logits: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Mean predictive entropy over positions whose *next* token is inside ``mask``."""
    logits = logits[..., :-1, :]
    m = mask[..., 1:]
    logp = logits.log_softmax(dim=-1)
    ent = -(logp.exp() * logp).sum(dim=-1)
    m = m.to(ent.dtype)
    return ((ent * m).sum() / m.sum().clamp(min=1)).detach()


def mean_token_accuracy(logits: torch.Tensor, labels: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    preds = logits[..., :-1, :].argmax(dim=-1)
    m = mask[..., 1:]
    correct = (preds == labels[..., 1:]) & m.bool()
    return (correct.sum() / m.to(logits.dtype).sum().clamp(min=1)).detach()
