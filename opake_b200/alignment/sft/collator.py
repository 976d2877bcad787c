"""Language-modelling collator (packages/opake-alignment/src/opake/api/alignment/sft/collator/
_language_modeling.py:48-236): keep-start truncation, right padding, ``-100`` labels on padding and, with
``completion_only_loss``, on prompt tokens."""
from __future__ import annotations

from typing import Callable, NotRequired, TypedDict

import torch

IGNORE_INDEX = -100
__all__ = ["LMExample", "LMBatch", "language_modeling_collator"]


class LMExample(TypedDict):
    input_ids: list[int]
    completion_mask: NotRequired[list[int]]


class LMBatch(TypedDict):
    input_ids: torch.Tensor
    attention_mask: torch.Tensor
    labels: torch.Tensor
    completion_mask: NotRequired[torch.Tensor]


def language_modeling_collator(pad_token_id: int, max_length: int, *, completion_only_loss: bool = False,
                               pad_to_multiple_of: int | None = None) -> Callable[[list[LMExample]], LMBatch]:
    def collate(examples: list[LMExample]) -> LMBatch:
        if not examples:
            empty = torch.zeros((0, 0), dtype=torch.long)
            return {"input_ids": empty, "attention_mask": empty, "labels": empty}
        ids = [list(ex["input_ids"][:max_length]) for ex in examples]
        masks = [ex.get("completion_mask") for ex in examples]
        masks = [None if m is None else list(m[:max_length]) for m in masks]
        has_mask = any(m is not None for m in masks)
        L = min(max(len(x) for x in ids), max_length)
        if pad_to_multiple_of and pad_to_multiple_of > 1 and L % pad_to_multiple_of:
            L += pad_to_multiple_of - L % pad_to_multiple_of
        B = len(ids)
        input_ids = torch.full((B, L), pad_token_id, dtype=torch.long)
        attention = torch.zeros((B, L), dtype=torch.long)
        labels = torch.full((B, L), IGNORE_INDEX, dtype=torch.long)
        cmask = torch.zeros((B, L), dtype=torch.long) if has_mask else None
        for i, (x, m) in enumerate(zip(ids, masks)):
            n = len(x)
            row = torch.tensor(x, dtype=torch.long)
            input_ids[i, :n] = row
            attention[i, :n] = 1
            labels[i, :n] = row
            if cmask is not None:
                if m is None:
                    cmask[i, :n] = 1          # an example without a mask is fully supervised
                else:
                    mt = torch.tensor(m, dtype=torch.long)
                    cmask[i, :n] = mt
                    if completion_only_loss:
                        labels[i, :n][mt == 0] = IGNORE_INDEX
        out: LMBatch = {"input_ids": input_ids, "attention_mask": attention, "labels": labels}
        if cmask is not None:
            out["completion_mask"] = cmask
        return out

    return collate
