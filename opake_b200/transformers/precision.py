"""Precision helpers (packages/opake-transformers/src/opake/api/transformers/trainer/_precision.py:24-65)."""
from __future__ import annotations

import contextlib

import torch

__all__ = ["eval_dtype", "autocast_context"]


def eval_dtype(args) -> torch.dtype | None:
    """dtype the model is cast to for evaluation (``bf16_full_eval``), else ``None`` (keep training dtype)."""
    return torch.bfloat16 if getattr(args, "bf16_full_eval", False) else None


def autocast_context(args, device: torch.device):
    if getattr(args, "bf16", False) and device.type in ("cuda", "cpu"):
        return torch.autocast(device_type=device.type, dtype=torch.bfloat16)
    return contextlib.nullcontext()
