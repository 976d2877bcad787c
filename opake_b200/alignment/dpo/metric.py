"""Reward telemetry for preference training (packages/opake-alignment/src/opake/api/alignment/dpo/metric/
_reward.py:17-54). Batch means of non-private quantities: log them only from evaluation data or treat as leakage."""
from __future__ import annotations

import torch

__all__ = ["reward_metrics"]


def reward_metrics(chosen_logratio: torch.Tensor, rejected_logratio: torch.Tensor, *, beta: float) -> dict:
    return {
        "rewards/chosen": (beta * chosen_logratio).mean().detach(),
        "rewards/rejected": (beta * rejected_logratio).mean().detach(),
        "rewards/accuracies": (chosen_logratio > rejected_logratio).float().mean().detach(),
        "rewards/margins": (beta * (chosen_logratio - rejected_logratio)).mean().detach(),
    }
