"""Fused clip-and-sum of materialised per-example gradients (counterpart of ``fused_clip_sum``,
packages/opake-patches/src/opake/api/patches/kernels/_clip_sum.py:270-379).

``leaves`` are ``[B, ...]`` tensors (bf16 or fp32) as produced by ``vmap(grad)``. Two multi-tensor kernels do the
heavy passes (per-example squared norms; scaled, storage-rounded, summed gradients); the clip factors in between are
computed on the ``[B]`` vector with exactly the code of the portable path, so both paths agree bit for bit on the
factors and to fp32 summation order on the sums.
"""
from __future__ import annotations

import struct
from typing import Sequence

import torch

from . import _lib

__all__ = ["fused_clip_sum", "supported"]

_TABLES: dict = {}


def supported(leaves: Sequence[torch.Tensor]) -> bool:
    return bool(leaves) and all(l.is_cuda and l.dtype in (torch.bfloat16, torch.float32) and l.dim() >= 1 for l in leaves) \
        and leaves[0].shape[0] <= 65535


def _tile_table(leaves, outs):
    lib = _lib.lib()
    tile = lib.opk_clip_sum_tile()
    key = tuple((l.data_ptr(), o.data_ptr(), l[0].numel(), l.dtype) for l, o in zip(leaves, outs))
    hit = _TABLES.get(key)
    if hit is not None:
        return hit
    assert lib.opk_clip_sum_desc_bytes() == 40
    blob = bytearray()
    n_tiles = 0
    for l, o in zip(leaves, outs):
        n = l[0].numel()
        for off in range(0, n, tile):
            blob += struct.pack("<QQqqii", l.data_ptr(), o.data_ptr(), n, off, int(l.dtype == torch.bfloat16), 0)
            n_tiles += 1
    table = torch.frombuffer(blob, dtype=torch.uint8).to(leaves[0].device)
    if len(_TABLES) > 64:
        _TABLES.clear()
    _TABLES[key] = (table, n_tiles)
    return table, n_tiles


def fused_clip_sum(leaves: Sequence[torch.Tensor], clipping_norm: float, *, with_postsq: bool = False, out_dtypes=None):
    """Returns ``(sums, norms, clipped_mask, post_norms)``: per-leaf fp32 sums of the clipped examples, the ``[B]``
    pre-clip norms (fp64), which examples were clipped, and (``with_postsq``) the norms after clipping."""
    from ..engine.clipping import numerics as N
    lib = _lib.lib()
    leaves = [l.contiguous() for l in leaves]
    dev = leaves[0].device
    B = leaves[0].shape[0]
    outs = [torch.empty(l.shape[1:], dtype=torch.float32, device=dev) for l in leaves]
    if B == 0:
        for o in outs:
            o.zero_()
        z = torch.zeros(0, dtype=torch.float64, device=dev)
        return outs, z, z.bool(), (z if with_postsq else None)
    table, n_tiles = _tile_table(leaves, outs)
    st = _lib.stream_ptr(dev)
    partial = torch.empty(B, n_tiles, dtype=torch.float64, device=dev)
    _lib.check(lib.opk_clip_sumsq_partial(table.data_ptr(), n_tiles, B, partial.data_ptr(), st), "opk_clip_sumsq_partial")
    sq = partial.sum(1)
    factors, norms, mask = N.clip_factors(sq, clipping_norm, leaves)
    f_bf16 = f_fp32 = None
    for l, f in zip(leaves, factors):
        if l.dtype == torch.bfloat16 and f_bf16 is None:
            f_bf16 = f.to(torch.float32).contiguous()
        if l.dtype == torch.float32 and f_fp32 is None:
            f_fp32 = f.to(torch.float32).contiguous()
    post = torch.empty(B, n_tiles, dtype=torch.float64, device=dev) if with_postsq else None
    _lib.check(lib.opk_clip_apply_sum(table.data_ptr(), n_tiles, B, _lib.ptr(f_bf16), _lib.ptr(f_fp32), _lib.ptr(post), st),
               "opk_clip_apply_sum")
    if out_dtypes is not None:
        outs = [o.to(d) for o, d in zip(outs, out_dtypes)]
    return outs, norms, mask, (torch.sqrt(post.sum(1)) if with_postsq else None)
