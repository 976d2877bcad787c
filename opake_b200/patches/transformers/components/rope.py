"""Rotary-embedding replacement for the Hugging Face ``apply_rotary_pos_emb`` helpers (packages/opake-patches/src/
opake/api/patches/transformers/components/rope.py).

``apply_rotary_pos_emb(q, k, cos, sin)`` receives ``[B, H, T, hd]`` queries / keys and ``[B, T, hd]`` (or ``[T, hd]``)
tables. On CUDA bf16, when the tables do not depend on the batch index, queries and keys are rotated in ONE launch of
this package's rotate-half kernel over a fused ``[T, (Hq + Hk) * hd]`` buffer; everything else (CPU, per-example
position ids, partial rotary dimensions) takes the same formula in eager mode."""
from __future__ import annotations

import sys

import torch

from ...kernels.functions import native_rows, opake_rope_qk

__all__ = ["opake_apply_rotary_pos_emb", "apply_rope_patch", "make_rope_replacement", "rotate_half"]

_MARK = "_opake_rope"


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def _eager(q, k, cos, sin, unsqueeze_dim):
    c, s = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return q * c + rotate_half(q) * s, k * c + rotate_half(k) * s


def _fast_path_ok(q, k, cos, unsqueeze_dim) -> bool:
    hd = q.shape[-1]
    table_2d = cos.dim() == 2 or (cos.dim() == 3 and cos.shape[0] == 1)
    return bool(q.is_cuda and native_rows(q) and table_2d and cos.shape[-1] == hd and unsqueeze_dim == 1 and q.dim() == 4
                and q.shape[0] == 1 and k.dim() == 4 and hd % 2 == 0)


def _fused_rotate(q, k, cos, sin):
    hd = q.shape[-1]
    c2, s2 = cos.reshape(-1, hd), sin.reshape(-1, hd)
    T, hq, hk = q.shape[-2], q.shape[1], k.shape[1]
    # [T, hd/2, 2] cos / sin table of the rotate-half convention (both halves of cos / sin are equal)
    table = torch.stack((c2[:T, : hd // 2], s2[:T, : hd // 2]), dim=-1).float().contiguous()
    fused = torch.cat((q[0].transpose(0, 1).reshape(T, hq * hd), k[0].transpose(0, 1).reshape(T, hk * hd)), dim=-1)
    out = opake_rope_qk(fused, table, hq + hk, hd)
    q2 = out[:, : hq * hd].reshape(T, hq, hd).transpose(0, 1)[None]
    k2 = out[:, hq * hd:].reshape(T, hk, hd).transpose(0, 1)[None]
    return q2, k2


def opake_apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim: int = 1):
    """Rotate-half convention with full-width tables; anything else in eager mode."""
    if _fast_path_ok(q, k, cos, unsqueeze_dim):
        return _fused_rotate(q, k, cos, sin)
    return _eager(q, k, cos, sin, unsqueeze_dim)


setattr(opake_apply_rotary_pos_emb, _MARK, True)


def make_rope_replacement(original):
    """Fast path when it applies, the modeling module's OWN function otherwise (partial rotary dimensions, interleaved
    conventions and per-example position ids keep their stock semantics)."""

    def apply_rotary_pos_emb(q, k, cos, sin, *args, **kwargs):
        unsqueeze_dim = kwargs.get("unsqueeze_dim", args[1] if len(args) > 1 else 1)
        if _fast_path_ok(q, k, cos, unsqueeze_dim):
            return _fused_rotate(q, k, cos, sin)
        return original(q, k, cos, sin, *args, **kwargs)

    setattr(apply_rotary_pos_emb, _MARK, True)
    apply_rotary_pos_emb.__wrapped__ = original
    return apply_rotary_pos_emb


def apply_rope_patch(model) -> int:
    """Replaces ``apply_rotary_pos_emb`` in the modeling module(s) that define ``model``'s classes. Returns how many
    modules were changed."""
    seen, n = set(), 0
    for m in model.modules():
        mod = sys.modules.get(type(m).__module__)
        if mod is None or mod.__name__ in seen:
            continue
        seen.add(mod.__name__)
        fn = mod.__dict__.get("apply_rotary_pos_emb")
        if fn is not None and not getattr(fn, _MARK, False):
            mod.apply_rotary_pos_emb = make_rope_replacement(fn)
            n += 1
    return n
