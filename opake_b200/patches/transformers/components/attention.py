"""vmap-safe building blocks that replace Hugging Face sub-module forwards (packages/opake-patches/src/opake/api/
patches/transformers/components/*.py: attention.py:75-113,169,384,542; rms_norm, swiglu, geglu, rope, dropout,
kv_cache, batchify, cross_entropy.py:175; runtime/masking.py:253,415,626).

Under ``vmap(grad)`` a model sees ONE example with the batch dimension hidden, and several stock Hugging Face code
paths break there: data-dependent mask construction (``.item()``, boolean indexing), in-place KV-cache updates,
dropout without per-example randomness, attention kernels without batching rules. The replacements below are pure
functions of tensors with static control flow.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


__all__ = ["causal_mask", "sliding_window_mask", "vmap_sdpa_attention_forward", "eager_attention_forward",
           "softcapped_attention", "SoftcappedAttention", "softcapped_attention_recompute", "repeat_kv"]


def causal_mask(q_len: int, kv_len: int, device, dtype=torch.bool, attention_mask: torch.Tensor | None = None):
    """``[.., q_len, kv_len]`` boolean mask (True = attend) built from iota comparisons only."""
    qi = torch.arange(kv_len - q_len, kv_len, device=device)[:, None]
    ki = torch.arange(kv_len, device=device)[None, :]
    m = ki <= qi
    if attention_mask is not None:
        m = m & attention_mask[..., None, :].to(torch.bool)
    return m


def sliding_window_mask(q_len: int, kv_len: int, window: int, device, attention_mask: torch.Tensor | None = None):
    qi = torch.arange(kv_len - q_len, kv_len, device=device)[:, None]
    ki = torch.arange(kv_len, device=device)[None, :]
    m = (ki <= qi) & (ki > qi - window)
    if attention_mask is not None:
        m = m & attention_mask[..., None, :].to(torch.bool)
    return m


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[..., kv_heads, T, hd]`` -> ``[..., kv_heads * n_rep, T, hd]`` (expand + reshape, no data-dependent ops)."""
    if n_rep == 1:
        return x
    *lead, h, t, d = x.shape
    return x.unsqueeze(-3).expand(*lead, h, n_rep, t, d).reshape(*lead, h * n_rep, t, d)


def vmap_sdpa_attention_forward(module, query, key, value, attention_mask=None, dropout: float = 0.0, scaling: float | None = None,
                                is_causal: bool | None = None, sliding_window: int | None = None, **_kw):
    """Drop-in for the Hugging Face attention interface: ``[B, H, T, hd]`` in, ``([B, T, H, hd], None)`` out. Grouped
    heads are expanded explicitly and the mask is rebuilt from shapes, so the call is legal under vmap."""
    n_rep = query.shape[-3] // key.shape[-3]
    key, value = repeat_kv(key, n_rep), repeat_kv(value, n_rep)
    q_len, kv_len = query.shape[-2], key.shape[-2]
    mask = None
    causal = is_causal if is_causal is not None else (attention_mask is None and q_len > 1)
    if sliding_window is not None and sliding_window < kv_len:
        mask, causal = sliding_window_mask(q_len, kv_len, sliding_window, query.device), False
    elif attention_mask is not None:
        mask = attention_mask[..., :kv_len] if attention_mask.dtype == torch.bool else attention_mask[..., :kv_len]
        causal = False
    out = F.scaled_dot_product_attention(query, key, value, attn_mask=mask, dropout_p=0.0, is_causal=bool(causal), scale=scaling)
    return out.transpose(-3, -2).contiguous(), None


def eager_attention_forward(module, query, key, value, attention_mask=None, scaling: float | None = None, softcap: float | None = None,
                            sliding_window: int | None = None, **_kw):
    if softcap and attention_mask is None and not _kw.get("output_attentions") and query.shape[-2] == key.shape[-2]:
        # soft-capped training pass without padding: the recomputing function keeps no [H, T, T] tensor for the backward
        out = softcapped_attention_recompute(query, key, value, softcap, scaling, sliding_window)
        return out.transpose(-3, -2).contiguous(), None
    n_rep = query.shape[-3] // key.shape[-3]
    key, value = repeat_kv(key, n_rep), repeat_kv(value, n_rep)
    scale = scaling if scaling is not None else 1.0 / math.sqrt(query.shape[-1])
    s = torch.matmul(query, key.transpose(-1, -2)) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    q_len, kv_len = query.shape[-2], key.shape[-2]
    # local-attention layers (Gemma-2 / Gemma-3, Mistral, ...) pass their window; the library may hand over no mask at
    # all for an unpadded batch, so the window is rebuilt here from the shapes
    if sliding_window is not None and sliding_window < kv_len:
        m = sliding_window_mask(q_len, kv_len, int(sliding_window), query.device)
    else:
        m = causal_mask(q_len, kv_len, query.device)
    if attention_mask is not None:
        m = m & (attention_mask[..., :kv_len] if attention_mask.dtype == torch.bool else attention_mask[..., :kv_len] == 0)
    s = s.masked_fill(~m, torch.finfo(s.dtype).min)
    p = torch.softmax(s.float(), dim=-1).to(query.dtype)
    return torch.matmul(p, value).transpose(-3, -2).contiguous(), p


def softcapped_attention(query, key, value, softcap: float, scaling: float | None = None, chunk: int = 1024):
    """Gemma-2 style attention with logit soft-capping, computed over query chunks so that the ``[T, T]`` score matrix
    never exists at once (sequence length is scaled by chunking, not by sequence parallelism)."""
    outs = []
    kv_len = key.shape[-2]
    scale = scaling if scaling is not None else 1.0 / math.sqrt(query.shape[-1])
    n_rep = query.shape[-3] // key.shape[-3]
    key, value = repeat_kv(key, n_rep), repeat_kv(value, n_rep)
    for lo in range(0, query.shape[-2], chunk):
        q = query[..., lo:lo + chunk, :]
        s = torch.matmul(q, key.transpose(-1, -2)) * scale
        s = softcap * torch.tanh(s / softcap)
        qi = torch.arange(lo, lo + q.shape[-2], device=q.device)[:, None] + (kv_len - query.shape[-2])
        s = s.masked_fill(torch.arange(kv_len, device=q.device)[None, :] > qi, torch.finfo(s.dtype).min)
        outs.append(torch.matmul(torch.softmax(s.float(), -1).to(q.dtype), value))
    return torch.cat(outs, dim=-2)


class SoftcappedAttention(torch.autograd.Function):
    """Causal attention with soft-capped logits (``cap * tanh(s / cap)``, Gemma-2) whose backward RECOMPUTES the scores
    chunk by chunk instead of keeping them: autograd through :func:`softcapped_attention` saves, per layer, the
    ``[H, T, T]`` pre-cap scores, their tanh and the probabilities; this function saves q, k, v, the output and one
    log-sum-exp per row. Inputs ``[..., H, T, hd]`` (grouped heads already expanded), optional sliding ``window``.
    Works under ``vmap`` / ``vmap(grad)`` through the generated batching rule (all internals are batched tensor ops)."""

    generate_vmap_rule = True

    @staticmethod
    def forward(query, key, value, softcap: float, scale: float, window: int, chunk: int):
        kv_len, q_len = key.shape[-2], query.shape[-2]
        outs, lses = [], []
        for lo in range(0, q_len, chunk):
            q = query[..., lo:lo + chunk, :]
            z = _capped_scores(q, key, softcap, scale, lo + kv_len - q_len, window)
            lse = torch.logsumexp(z, dim=-1)
            outs.append(torch.matmul(torch.exp(z - lse[..., None]).to(value.dtype), value))
            lses.append(lse)
        return torch.cat(outs, dim=-2), torch.cat(lses, dim=-1)

    @staticmethod
    def setup_context(ctx, inputs, output):
        query, key, value, softcap, scale, window, chunk = inputs
        out, lse = output
        ctx.save_for_backward(query, key, value, out, lse)
        ctx.cfg = (softcap, scale, window, chunk)
        ctx.mark_non_differentiable(lse)

    @staticmethod
    def backward(ctx, d_out, _d_lse):
        query, key, value, out, lse = ctx.saved_tensors
        softcap, scale, window, chunk = ctx.cfg
        kv_len, q_len = key.shape[-2], query.shape[-2]
        dq = []
        dk = torch.zeros_like(key, dtype=torch.float32)
        dv = torch.zeros_like(value, dtype=torch.float32)
        for lo in range(0, q_len, chunk):
            sl = slice(lo, lo + chunk)
            q, do = query[..., sl, :], d_out[..., sl, :]
            raw = torch.matmul(q.float(), key.float().transpose(-1, -2)) * scale
            th = torch.tanh(raw / softcap)
            z = _mask_scores(softcap * th, q.shape[-2], kv_len, lo + kv_len - q_len, window)
            p = torch.exp(z - lse[..., sl, None])
            dv = dv + torch.matmul(p.transpose(-1, -2), do.float())
            dp = torch.matmul(do.float(), value.float().transpose(-1, -2))
            delta = (do.float() * out[..., sl, :].float()).sum(-1, keepdim=True)
            ds = p * (dp - delta) * (1.0 - th * th) * scale           # through softmax, then cap * tanh(raw / cap)
            dq.append(torch.matmul(ds, key.float()).to(query.dtype))
            dk = dk + torch.matmul(ds.transpose(-1, -2), q.float())
        return torch.cat(dq, dim=-2), dk.to(key.dtype), dv.to(value.dtype), None, None, None, None


def _mask_scores(z, q_len: int, kv_len: int, q_offset: int, window: int):
    qi = torch.arange(q_offset, q_offset + q_len, device=z.device)[:, None]
    ki = torch.arange(kv_len, device=z.device)[None, :]
    keep = ki <= qi
    if window and window < kv_len:
        keep = keep & (ki > qi - window)
    return z.masked_fill(~keep, float("-inf"))


def _capped_scores(q, key, softcap: float, scale: float, q_offset: int, window: int):
    raw = torch.matmul(q.float(), key.float().transpose(-1, -2)) * scale
    return _mask_scores(softcap * torch.tanh(raw / softcap), q.shape[-2], key.shape[-2], q_offset, window)


def softcapped_attention_recompute(query, key, value, softcap: float, scaling: float | None = None, sliding_window: int | None = None,
                                   chunk: int = 1024):
    """Functional front end of :class:`SoftcappedAttention` (expands grouped heads, fills defaults)."""
    n_rep = query.shape[-3] // key.shape[-3]
    key, value = repeat_kv(key, n_rep), repeat_kv(value, n_rep)
    scale = scaling if scaling is not None else 1.0 / math.sqrt(query.shape[-1])
    out, _ = SoftcappedAttention.apply(query, key, value, float(softcap), float(scale), int(sliding_window or 0), int(chunk))
    return out
