"""Cross-rank audit of optimizer state (packages/opake-optimizers/src/opake/api/optimizers/distributed.py:186-231):
replicated data-parallel ranks must hold identical moments; a (sum, sum of squares, min, max) fingerprint per leaf is
compared with one reduction."""
from __future__ import annotations

from typing import Any

from ..engine import distributed as D
from ..engine.pytree import tree_leaves


def _tensors(obj: Any):
    import dataclasses

    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        for f in dataclasses.fields(obj):
            yield from _tensors(getattr(obj, f.name))
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _tensors(v)
    elif isinstance(obj, dict):
        for k in sorted(obj, key=str):
            yield from _tensors(obj[k])
    else:
        import torch

        if isinstance(obj, torch.Tensor):
            yield obj


def sync_optimizer_state(state: Any, *, atol: float = 0.0) -> Any:
    D.assert_pytree_equal(list(_tensors(state)), name="optimizer state", atol=atol)
    return state


__all__ = ["sync_optimizer_state"]
