"""Prompt extraction for preference datasets (packages/opake-alignment/src/opake/api/alignment/dpo/data/_prompt.py)."""
from __future__ import annotations

__all__ = ["extract_prompt"]


def extract_prompt(example: dict) -> dict:
    """Splits the longest common prefix of ``chosen`` and ``rejected`` (lists of turns or tokens) off as ``prompt``."""
    if "prompt" in example or "chosen" not in example or "rejected" not in example:
        return example
    chosen, rejected = example["chosen"], example["rejected"]
    n = 0
    for c, r in zip(chosen, rejected):
        if c != r:
            break
        n += 1
    return {**example, "prompt": chosen[:n], "chosen": chosen[n:], "rejected": rejected[n:]}
