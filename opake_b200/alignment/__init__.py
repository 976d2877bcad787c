"""Functional primitives for DP-safe supervised fine-tuning and preference learning (counterpart of the
``opake.alignment`` namespace, packages/opake-alignment/src/opake/alignment/__init__.py)."""
from . import data, dpo, metric, sft

__all__ = ["data", "dpo", "metric", "sft"]
