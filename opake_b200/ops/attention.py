"""Causal grouped-query attention over a fused ``[T, (H + 2*KV) * hd]`` projection buffer.

``impl="flash"`` runs the hand-written tcgen05 kernels (csrc/kernels/attention_sm100.cu); ``impl="sdpa"`` is a
library stopgap (PyTorch scaled_dot_product_attention) kept only as a numerical oracle and for shapes the native
kernel does not cover. The reference calls the library through vmap-safe wrappers
(packages/opake-patches/src/opake/api/patches/transformers/components/attention.py:75-113).
"""
from __future__ import annotations

import torch

from . import _lib


def _split(qkv: torch.Tensor, H: int, KV: int, hd: int):
    T = qkv.shape[0]
    q = qkv[:, : H * hd].view(T, H, hd)
    k = qkv[:, H * hd : (H + KV) * hd].view(T, KV, hd)
    v = qkv[:, (H + KV) * hd :].view(T, KV, hd)
    return q, k, v


def have_flash() -> bool:
    L = _lib.lib()
    return hasattr(L, "opk_attn_fwd") and hasattr(L, "opk_attn_bwd")


def attention_fwd(qkv: torch.Tensor, H: int, KV: int, hd: int, impl: str = "auto", out: torch.Tensor | None = None):
    """Returns ``(out [T, H*hd] bf16, ctx)``; ``ctx`` is what :func:`attention_bwd` needs."""
    if impl == "auto":
        impl = "flash" if (have_flash() and hd in (64, 128)) else "sdpa"
    if impl == "flash":
        from .flash import flash_fwd

        out, lse = flash_fwd(qkv, H, KV, hd, out=out)
        return out, ("flash", lse)
    q, k, v = _split(qkv, H, KV, hd)
    qh = q.transpose(0, 1).unsqueeze(0).detach().requires_grad_()
    kh = k.transpose(0, 1).unsqueeze(0).detach().requires_grad_()
    vh = v.transpose(0, 1).unsqueeze(0).detach().requires_grad_()
    with torch.enable_grad():
        o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=(H != KV))
    res = o.detach().squeeze(0).transpose(0, 1).reshape(qkv.shape[0], H * hd)
    if out is not None:
        out.copy_(res)
    else:
        out = res.contiguous()
    return out, ("sdpa", (o, qh, kh, vh))


def attention_bwd(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, hd: int,
                  dqkv: torch.Tensor | None = None) -> torch.Tensor:
    """Gradient with respect to the fused projection buffer, same layout as ``qkv``."""
    kind, saved = ctx
    T = qkv.shape[0]
    if dqkv is None:
        dqkv = torch.empty_like(qkv)
    if kind == "flash":
        from .flash import flash_bwd

        return flash_bwd(dout, qkv, out, saved, H, KV, hd, dqkv)
    o, qh, kh, vh = saved
    go = dout.view(T, H, hd).transpose(0, 1).unsqueeze(0)
    dq, dk, dv = torch.autograd.grad(o, (qh, kh, vh), go)
    dqv, dkv, dvv = _split(dqkv, H, KV, hd)
    dqv.copy_(dq.squeeze(0).transpose(0, 1))
    dkv.copy_(dk.squeeze(0).transpose(0, 1))
    dvv.copy_(dv.squeeze(0).transpose(0, 1))
    return dqkv
