"""Privacy-preserving clip arithmetic on batches of per-example pytrees.

The rule set is the reference's (packages/opake-engine/src/opake/api/engine/clipping/_pytree.py:111-204,245-314,
422-507,560-649):

1. non-finite entries are replaced by zero;
2. per-example squared norms accumulate in float64 (leaves are squared in fp32 for bf16/fp16 storage), long leaves
   in 2048-element blocks;
3. the clip factor ``C / norm`` is *shrunk* by the worst-case rounding of the norm accumulation, of the multiply and
   of the store, so that the norm of the stored clipped value cannot exceed ``C``; it is clamped to 1 afterwards
   (unclipped examples pass unchanged), non-finite factors become 0;
4. after the store, subnormal results that rounded away from zero are flushed to zero.

Everything here is batched: leaves carry a leading example dimension ``[B, ...]`` and factors are ``[B]`` tensors,
so the same code serves vmap outputs on CPU and GPU. On CUDA the fused path (:mod:`opake_b200.ops.clip_sum`) does
steps 2-4 in three launches for the whole tree.
"""
from __future__ import annotations

import math
from collections.abc import Sequence

import torch

_BLOCK = 2048
_BLOCK_THRESHOLD = 4096


def acc_dtype_of(dtype: torch.dtype) -> torch.dtype:
    if dtype in (torch.bfloat16, torch.float16):
        return torch.float32
    return torch.promote_types(dtype, torch.float32) if dtype.is_floating_point else torch.float32


def sq_dtype_for(device: torch.device) -> torch.dtype:
    return torch.float32 if device.type == "mps" else torch.float64


def sanitize(t: torch.Tensor) -> torch.Tensor:
    return torch.nan_to_num(t, nan=0.0, posinf=0.0, neginf=0.0)


def per_example_sq(leaf: torch.Tensor, sq_dtype: torch.dtype) -> torch.Tensor:
    """``[B]`` squared L2 norms of a ``[B, ...]`` leaf (fp32 square, fp64 two-stage sum)."""
    B = leaf.shape[0]
    x = leaf.reshape(B, -1).to(acc_dtype_of(leaf.dtype))
    n = x.shape[1]
    sq = (x * x)
    if n > _BLOCK_THRESHOLD:
        pad = (-n) % _BLOCK
        if pad:
            sq = torch.nn.functional.pad(sq, (0, pad))
        return sq.view(B, -1, _BLOCK).sum(-1, dtype=sq_dtype).sum(-1, dtype=sq_dtype)
    return sq.sum(-1, dtype=sq_dtype)


def reduction_length(numel: int) -> int:
    return _BLOCK + math.ceil(numel / _BLOCK) if numel > _BLOCK_THRESHOLD else numel


def norm_roundoff(leaves: Sequence[torch.Tensor], sq_dtype: torch.dtype) -> float:
    """Relative error bound of the computed norm (per example): (u_acc + (leaves + reductions) * u_sq) / 2."""
    if not leaves:
        return 0.0
    u_acc = max(torch.finfo(acc_dtype_of(l.dtype)).eps for l in leaves) / 2
    u_sq = torch.finfo(sq_dtype).eps / 2
    widest = max(reduction_length(l[0].numel() if l.dim() > 0 else 1) for l in leaves)
    return (u_acc + (max(len(leaves), 1) + widest) * u_sq) / 2


def guard_factor(ratio: torch.Tensor, store: torch.dtype, multiply: torch.dtype, roundoff: float,
                 clamp_to_one: bool = True) -> torch.Tensor:
    """Conservative clip factor for leaves stored as ``store`` and multiplied in ``multiply``."""
    fs, fm = torch.finfo(store), torch.finfo(multiply)
    rounding = fs.eps if store == multiply else fs.eps / 2 + fm.eps
    s = ratio * (1.0 - rounding - 2.0 * roundoff) - fs.smallest_normal * fs.eps
    if clamp_to_one:
        s = torch.clamp(s, max=1.0)
    s = torch.where(torch.isfinite(s), s, torch.zeros_like(s))
    return torch.clamp(s, min=0.0)


def scale_leaf(leaf: torch.Tensor, factor: torch.Tensor) -> torch.Tensor:
    """``leaf[b] * factor[b]`` stored in the leaf dtype with the subnormal flush."""
    mult = torch.promote_types(leaf.dtype, acc_dtype_of(leaf.dtype))
    f = factor.to(mult).view(-1, *([1] * (leaf.dim() - 1)))
    scaled = leaf.to(mult) * f
    stored = scaled.to(leaf.dtype)
    tiny = torch.finfo(leaf.dtype).smallest_normal
    back = stored.to(mult)
    bad = (back.abs() <= tiny) & (back.abs() > scaled.abs())
    return torch.where(bad, torch.zeros_like(stored), stored)


def clip_factors(sq_norms: torch.Tensor, clipping_norm: float, leaves: Sequence[torch.Tensor], *, auto: bool = False,
                 gamma: float = 0.01):
    """Per-leaf ``[B]`` factors from per-example squared norms.

    Returns ``(factors per leaf, norms, clipped mask)``. ``C = 0`` gives zeros, ``C = inf`` passes everything,
    zero norms are left unchanged (fixed clipping).
    """
    sq_dtype = sq_norms.dtype
    norms = torch.sqrt(sq_norms)
    C = max(float(clipping_norm), 0.0)
    ro = norm_roundoff(leaves, sq_dtype)
    if auto:
        ratio = C / (norms + gamma)
    else:
        ratio = torch.where(norms > 0, C / norms, torch.full_like(norms, math.inf))
    out = []
    for l in leaves:
        mult = torch.promote_types(l.dtype, acc_dtype_of(l.dtype))
        if math.isinf(C) and not auto:
            out.append(torch.ones_like(norms))
            continue
        f = guard_factor(ratio, l.dtype, mult, ro, clamp_to_one=not auto)
        if not auto:
            f = torch.where(norms == 0, torch.ones_like(f), f)
        if C == 0.0:
            f = torch.zeros_like(f)
        out.append(f)
    clipped_mask = norms > C if not auto else torch.ones_like(norms, dtype=torch.bool)
    return out, norms, clipped_mask
