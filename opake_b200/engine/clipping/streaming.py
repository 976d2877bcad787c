"""Portable streaming clip-and-sum: two passes over the per-example gradient leaves, one leaf at a time.

Pass 1 reduces every leaf to its per-example squared norms (accumulated across leaves in the wide ``sq`` dtype), from
which the guarded clip factors follow. Pass 2 scales and batch-reduces leaf by leaf, so at no point does a second,
scaled copy of the whole per-example gradient exist: the extra memory is one leaf. This is the path for everything the
fused CUDA backend does not take (CPU tensors, AUTO-S, a custom scale function, the private second-moment stream, an
explicit compute dtype); behaviour of packages/opake-engine/src/opake/api/engine/clipping/_streaming.py:39-185, backend
choice of _clipped_fun.py:795-804.
"""
from __future__ import annotations

from typing import Callable

import torch

from . import numerics as N
from .kernel_backend import get_fused_clip_backend

__all__ = ["resolve_stream_impl", "stream_clip_and_sum"]


def resolve_stream_impl(leaves, clipping_norm, *, scale_fn=None, builtin_kind: str = "fixed", second_moment: bool = False,
                        compute_dtype=None) -> str:
    """``"fused"`` (registered multi-tensor CUDA backend) or ``"stream"`` (this module). The fused backend is used only
    for a scalar clipping norm, the built-in fixed scale, no private second moment and the default reduction dtype, on
    leaves it declares support for."""
    fused = get_fused_clip_backend()
    if (fused is not None and scale_fn is None and builtin_kind != "auto" and not second_moment and compute_dtype is None
            and not isinstance(clipping_norm, torch.Tensor) and isinstance(clipping_norm, (int, float)) and fused.supported(leaves)):
        return "fused"
    return "stream"


def stream_clip_and_sum(leaves: list[torch.Tensor], clipping_norm, *, scale_fn: Callable | None = None, auto: bool = False,
                        gamma: float = 0.01, second_moment: bool = False, compute_dtype=None, with_postsq: bool = False):
    """``leaves``: per-example gradients ``[B, ...]``. Returns ``(sums, squared sums or None, norms, clipped mask,
    clipped norms or None)``; ``sums[i] = sum_b stored(scale_b * leaves[i][b])`` in the accumulation dtype."""
    dev = leaves[0].device
    sqd = compute_dtype if compute_dtype is not None else N.sq_dtype_for(dev)
    # ---- pass 1: per-example squared norms, leaf by leaf
    sq = None
    for leaf in leaves:
        part = N.per_example_sq(leaf, sqd)
        sq = part if sq is None else sq + part
    if scale_fn is not None:
        norms = torch.sqrt(sq)
        f = scale_fn(norms)
        factors, mask = [f] * len(leaves), norms > float(clipping_norm)
    else:
        factors, norms, mask = N.clip_factors(sq, clipping_norm, leaves, auto=auto, gamma=gamma)
    # ---- pass 2: scale + batch-reduce, one leaf at a time
    sums, sq_sums, post = [], ([] if second_moment else None), None
    for leaf, f in zip(leaves, factors):
        scaled = N.scale_leaf(leaf, f)
        acc_dt = N.acc_dtype_of(scaled.dtype)
        sums.append(scaled.sum(0, dtype=acc_dt))
        if second_moment:
            sq_sums.append((scaled.to(acc_dt) ** 2).sum(0))
        if with_postsq:
            part = N.per_example_sq(scaled, sqd)
            post = part if post is None else post + part
        del scaled
    return sums, sq_sums, norms, mask, (torch.sqrt(post) if post is not None else None)
