"""Supervised fine-tuning losses, one value per example (packages/opake-alignment/src/opake/api/alignment/sft/loss/
_nll.py:43-124, _dft.py:30-147). Each loss divides by that example's own number of supervised tokens, so an
example's gradient never depends on the rest of the batch (the property DP clipping needs)."""
from __future__ import annotations

import torch

from ..logprob import _compute_dtype, selective_log_softmax

IGNORE_INDEX = -100
__all__ = ["nll_loss", "fused_nll_loss", "dft_loss", "fused_dft_loss"]


def _shift(logits, labels):
    sl = logits[..., :-1, :]
    lab = labels[..., 1:]
    valid = lab != IGNORE_INDEX
    return sl, lab.clamp(min=0), valid


def nll_loss(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    sl, lab, valid = _shift(logits, labels)
    logp = selective_log_softmax(sl, lab)
    acc = _compute_dtype(logp)
    n = valid.sum(-1).clamp(min=1)
    return (-logp * valid.to(sl.dtype)).to(acc).sum(-1) / n.to(acc)


def dft_loss(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Dynamic fine-tuning: every token's NLL is weighted by its own detached probability."""
    sl, lab, valid = _shift(logits, labels)
    logp = selective_log_softmax(sl, lab)
    per_token = -logp.exp().detach() * logp
    acc = _compute_dtype(per_token)
    n = valid.sum(-1).clamp(min=1)
    return (per_token * valid.to(sl.dtype)).to(acc).sum(-1) / n.to(acc)


def _fused(hidden_states, lm_head_weight, labels, token_scaling: bool):
    from ...ops.lce import opake_linear_cross_entropy_loss
    total = opake_linear_cross_entropy_loss(hidden_states, lm_head_weight, labels, use_token_scaling=token_scaling)
    n = (labels[..., 1:] != IGNORE_INDEX).sum(-1).clamp(min=1)
    return total / n


def fused_nll_loss(hidden_states, lm_head_weight, labels) -> torch.Tensor:
    return _fused(hidden_states, lm_head_weight, labels, False)


def fused_dft_loss(hidden_states, lm_head_weight, labels) -> torch.Tensor:
    return _fused(hidden_states, lm_head_weight, labels, True)
