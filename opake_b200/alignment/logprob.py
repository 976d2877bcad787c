"""Per-sequence log-probabilities of completions (packages/opake-alignment/src/opake/api/alignment/logprob/
_sequence.py:38-183, _gather.py:17-54)."""
from __future__ import annotations

import math

import torch

from ..base.exceptions import ConfigurationError

__all__ = ["selective_log_softmax", "sequence_logp", "fused_sequence_logp"]


def _compute_dtype(t: torch.Tensor) -> torch.dtype:
    return torch.promote_types(t.dtype, torch.float32)


def selective_log_softmax(logits: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[..., indices]`` without keeping the full log-softmax: ``logit[idx] - logsumexp``."""
    picked = torch.gather(logits, dim=-1, index=indices.unsqueeze(-1)).squeeze(-1)
    return picked - torch.logsumexp(logits, dim=-1)


def _ld_weight(target_mask, shared_prefix_len, alpha, dtype, device):
    pos = target_mask.to(torch.bool).cumsum(dim=-1)
    prefix = shared_prefix_len
    if isinstance(prefix, torch.Tensor):
        while prefix.ndim < pos.ndim:
            prefix = prefix.unsqueeze(-1)
    is_prefix = (pos >= 1) & (pos <= prefix)
    one = torch.ones((), dtype=dtype, device=device)
    return torch.where(is_prefix, one, torch.full((), alpha, dtype=dtype, device=device))


def sequence_logp(logits, input_ids, completion_mask, *, ld_alpha: float | None = None, shared_prefix_len=None,
                  length_normalized: bool = False) -> torch.Tensor:
    """Sum (or mean) over completion tokens of ``log p(token_{t+1} | prefix_t)``; shapes ``(..., L, V)`` / ``(..., L)``.

    With ``ld_alpha`` (LD-DPO) completion tokens beyond the first ``shared_prefix_len`` are weighted by ``ld_alpha``.
    """
    shifted = logits[..., :-1, :]
    targets = input_ids[..., 1:]
    mask = completion_mask[..., 1:]
    per_token = selective_log_softmax(shifted, targets)
    weight = mask.to(shifted.dtype)
    if ld_alpha is not None:
        if not math.isfinite(ld_alpha) or not 0.0 <= ld_alpha <= 1.0:
            raise ConfigurationError(f"ld_alpha (LD-DPO) must be finite and in [0, 1], got {ld_alpha}")
        if shared_prefix_len is None:
            raise ConfigurationError("ld_alpha (LD-DPO) requires shared_prefix_len")
        weight = weight * _ld_weight(mask, shared_prefix_len, ld_alpha, per_token.dtype, per_token.device)
    acc = _compute_dtype(per_token)
    logp = (per_token * weight).to(acc).sum(dim=-1)
    if length_normalized:
        logp = logp / mask.to(torch.bool).sum(-1).clamp(min=1).to(acc)
    return logp


def fused_sequence_logp(hidden_states, lm_head_weight, input_ids, completion_mask, *,
                        length_normalized: bool = False) -> torch.Tensor:
    """Same quantity from the last hidden states: the vocabulary projection and the log-softmax run inside the fused
    linear cross-entropy kernel, so ``(L, V)`` logits are never stored."""
    from ..ops.lce import opake_linear_cross_entropy_loss
    labels = torch.where(completion_mask.to(torch.bool), input_ids, torch.full_like(input_ids, -100))
    logp = -opake_linear_cross_entropy_loss(hidden_states, lm_head_weight, labels)
    if length_normalized:
        logp = logp / completion_mask[..., 1:].sum(-1).clamp(min=1).to(logp.dtype)
    return logp
