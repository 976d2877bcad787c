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

from ..kernels.functions import opake_geglu, opake_rms_norm, opake_swiglu

__all__ = ["causal_mask", "sliding_window_mask", "vmap_sdpa_attention_forward", "eager_attention_forward",
           "softcapped_attention", "patched_rms_norm_forward", "patched_gated_mlp_forward", "disable_dropout",
           "disable_kv_cache", "repeat_kv"]


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


def patched_rms_norm_forward(self, hidden_states):
    """Forward for ``*RMSNorm`` modules: fused kernel on CUDA bf16, same formula elsewhere. Modules that store
    ``weight - 1`` (Gemma) are recognised by ``_opake_offset``."""
    eps = getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6))
    return opake_rms_norm(hidden_states, self.weight, eps, getattr(self, "_opake_offset", 0.0))


def patched_gated_mlp_forward(self, x):
    act = getattr(self, "_opake_act", "silu")
    g, u = self.gate_proj(x), self.up_proj(x)
    return self.down_proj(opake_swiglu(g, u) if act == "silu" else opake_geglu(g, u, approximate=act))


def disable_dropout(model) -> int:
    """Sets every dropout probability to zero (per-example randomness under vmap is not defined for module dropout)."""
    n = 0
    for m in model.modules():
        if isinstance(m, torch.nn.Dropout) and m.p:
            m.p, n = 0.0, n + 1
    cfg = getattr(model, "config", None)
    for name in ("attention_dropout", "hidden_dropout", "resid_pdrop", "embd_pdrop", "attn_pdrop", "dropout"):
        if cfg is not None and isinstance(getattr(cfg, name, None), float) and getattr(cfg, name):
            setattr(cfg, name, 0.0)
    return n


def disable_kv_cache(model) -> None:
    cfg = getattr(model, "config", None)
    if cfg is not None and getattr(cfg, "use_cache", False):
        cfg.use_cache = False
