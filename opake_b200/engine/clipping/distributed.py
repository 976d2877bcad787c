"""Cross-rank synchronisation of clipping results (packages/opake-engine/src/opake/api/engine/clipping/
_distributed.py:46-306).

After the clipped gradient sums have been all-reduced, two more things must agree on every rank:

* the per-example auxiliary outputs (loss values, gradient norms, clipped norms, user aux): every rank only saw its own
  shard of the logical batch, and logging / adaptive rules want the whole batch. The reference gathers each field with
  one ``all_gather_object`` (pickle over the control plane); here all tensor fields of one aux object travel in ONE
  padded tensor all-gather (plus one tiny all-gather of the per-rank batch sizes), which is what NCCL is good at.
* the clipping statistics (number clipped, batch size, clipping rate): sums of integers, then the rate is recomputed.

Fixed-norm clip states carry nothing rank-dependent and pass through; adaptive clipping has its own rule
(``dpsgd.clipping.sync_adaptive_clip_state``), registered with ``engine.distributed.sync``.
"""
from __future__ import annotations

import dataclasses
from typing import Any

import torch

from .. import distributed as D
from ..pytree import tree_flatten, tree_unflatten

__all__ = ["sync_clip_state", "gather_aux_fields", "sync_clipping_rate", "sync_clipping_aux"]


def sync_clip_state(state: Any) -> Any:
    """Fixed clip states are identical on every rank by construction: returned unchanged. Other states go through the
    handlers registered with ``engine.distributed.register_sync_type``."""
    from .core import FixedClipState

    if type(state) is FixedClipState or not D.is_distributed():
        return state
    return D.sync(state)


def _gather_rows(rows: torch.Tensor, counts: list[int]) -> torch.Tensor:
    """All-gather of ``[B_local, F]`` row blocks with different ``B_local``: pad to the longest, gather, cut."""
    longest = max(counts)
    padded = rows.new_zeros((longest, rows.shape[1]))
    padded[: rows.shape[0]] = rows
    out = [torch.empty_like(padded) for _ in counts]
    torch.distributed.all_gather(out, padded)
    return torch.cat([o[:c] for o, c in zip(out, counts)])


def gather_aux_fields(aux: Any) -> Any:
    """Concatenates the per-example tensors of ``aux`` (a dataclass such as ``ClippedGradAux`` / ``ClippedFunAux``, or any
    pytree of ``[B_local, ...]`` tensors) over the ranks, in rank order. Non-tensor fields are kept from this rank.
    Every tensor field is flattened per example, packed side by side into one ``[B_local, F]`` float64 matrix and
    gathered in a single collective."""
    if not D.is_distributed() or aux is None:
        return aux
    fields = None
    if dataclasses.is_dataclass(aux) and not isinstance(aux, type):
        fields = {f.name: getattr(aux, f.name) for f in dataclasses.fields(aux)}
        tree = {k: v for k, v in fields.items() if k not in ("clipping_rate", "batch_size")}
    else:
        tree = aux
    leaves, td = tree_flatten(tree)
    slots = [i for i, l in enumerate(leaves) if isinstance(l, torch.Tensor) and l.dim() >= 1]
    if not slots:
        return aux
    local_b = leaves[slots[0]].shape[0]
    dev = leaves[slots[0]].device
    counts_t = torch.tensor([local_b], dtype=torch.int64, device=dev)
    all_counts = [torch.zeros_like(counts_t) for _ in range(D.get_world_size())]
    torch.distributed.all_gather(all_counts, counts_t)
    counts = [int(c.item()) for c in all_counts]
    widths = [int(leaves[i][0].numel()) if local_b else int(torch.tensor(leaves[i].shape[1:]).prod().item()) for i in slots]
    packed = torch.cat([leaves[i].reshape(local_b, -1).to(torch.float64) for i in slots], dim=1) if local_b else \
        torch.zeros((0, sum(widths)), dtype=torch.float64, device=dev)
    gathered = _gather_rows(packed, counts)
    col = 0
    for i, w in zip(slots, widths):
        src = leaves[i]
        leaves[i] = gathered[:, col : col + w].reshape(gathered.shape[0], *src.shape[1:]).to(src.dtype)
        col += w
    out_tree = tree_unflatten(td, leaves)
    if fields is None:
        return out_tree
    total = sum(counts)
    extra = {}
    if "batch_size" in fields:
        extra["batch_size"] = total
    return dataclasses.replace(aux, **out_tree, **extra)


def sync_clipping_rate(num_clipped, batch_size: int):
    """Global ``(num_clipped, batch_size, rate)`` from the local counts (integers are summed exactly; per-group counts
    arrive as a dict)."""
    if not D.is_distributed():
        rate = ({g: c / batch_size for g, c in num_clipped.items()} if isinstance(num_clipped, dict) else num_clipped / batch_size) \
            if batch_size else None
        return num_clipped, batch_size, rate
    total_b = int(D.reduce_scalar(int(batch_size), "sum"))
    if isinstance(num_clipped, dict):
        total_c = {g: float(D.reduce_scalar(float(c), "sum")) for g, c in sorted(num_clipped.items())}
        rate = {g: c / total_b for g, c in total_c.items()} if total_b else None
    else:
        total_c = float(D.reduce_scalar(float(num_clipped), "sum"))
        rate = total_c / total_b if total_b else None
    return total_c, total_b, rate


def sync_clipping_aux(aux: Any) -> Any:
    """``gather_aux_fields`` plus the global clipping rate for aux objects / ``ClippingStats`` that carry one."""
    from .core import ClippingStats

    if aux is None or not D.is_distributed():
        return aux
    if isinstance(aux, ClippingStats):
        c, b, r = sync_clipping_rate(aux.num_clipped, aux.batch_size)
        return ClippingStats(c, r, b)
    local_b = getattr(aux, "batch_size", 0)
    local_rate = getattr(aux, "clipping_rate", None)
    out = gather_aux_fields(aux)
    if local_rate is not None and dataclasses.is_dataclass(out):
        _, b, r = sync_clipping_rate(local_rate * local_b, local_b)
        out = dataclasses.replace(out, clipping_rate=r, batch_size=b)
    return out
