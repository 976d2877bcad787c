"""Preference-pair collator (packages/opake-alignment/src/opake/api/alignment/dpo/collator/_preference.py:40-229):
chosen and rejected sides are truncated (keep-start) and right-padded independently."""
from __future__ import annotations

import math
from typing import Callable, NotRequired, TypedDict

import torch

__all__ = ["PreferenceExample", "PreferenceBatch", "preference_collator"]


class PreferenceExample(TypedDict):
    chosen_input_ids: list[int]
    rejected_input_ids: list[int]
    chosen_completion_mask: list[int]
    rejected_completion_mask: list[int]
    ref_chosen_logps: NotRequired[float]
    ref_rejected_logps: NotRequired[float]


class PreferenceBatch(TypedDict):
    chosen_input_ids: torch.Tensor
    chosen_attention_mask: torch.Tensor
    chosen_completion_mask: torch.Tensor
    rejected_input_ids: torch.Tensor
    rejected_attention_mask: torch.Tensor
    rejected_completion_mask: torch.Tensor
    ref_chosen_logps: NotRequired[torch.Tensor]
    ref_rejected_logps: NotRequired[torch.Tensor]


def _pad(seqs, fill, length):
    out = torch.full((len(seqs), length), fill, dtype=torch.long)
    for i, s in enumerate(seqs):
        if s:
            out[i, :len(s)] = torch.tensor(s, dtype=torch.long)
    return out


def preference_collator(pad_token_id: int, max_length: int, *, pad_to_multiple_of: int | None = None
                        ) -> Callable[[list[PreferenceExample]], PreferenceBatch]:
    def side(batch, name):
        ids = [list(ex[f"{name}_input_ids"][:max_length]) for ex in batch]
        cm = [list(ex[f"{name}_completion_mask"][:max_length]) for ex in batch]
        L = max((len(s) for s in ids), default=0)
        if pad_to_multiple_of and pad_to_multiple_of > 1:
            L = math.ceil(L / pad_to_multiple_of) * pad_to_multiple_of
        attn = _pad([[1] * len(s) for s in ids], 0, L)
        return _pad(ids, pad_token_id, L), attn, _pad(cm, 0, L)

    def collate(batch: list[PreferenceExample]) -> PreferenceBatch:
        out: dict = {}
        for name in ("chosen", "rejected"):
            ids, attn, cm = side(batch, name)
            out[f"{name}_input_ids"], out[f"{name}_attention_mask"], out[f"{name}_completion_mask"] = ids, attn, cm
        for key in ("ref_chosen_logps", "ref_rejected_logps"):
            if all(key in ex for ex in batch):
                out[key] = torch.tensor([ex[key] for ex in batch], dtype=torch.float32)
        return out  # type: ignore[return-value]

    return collate
