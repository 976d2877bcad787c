"""Plain PyTorch (autograd) restatement of the decoder, used as the numerical oracle of the native runtime and as
the CPU execution path. Takes the same flat parameter views as :class:`DecoderRuntime`."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .config import DecoderConfig


def _rope(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    # x [T, heads, hd]; table [T, hd/2, 2]
    hd = x.shape[-1]
    cos = torch.cat([table[..., 0], table[..., 0]], -1)[:, None, :].to(x.dtype)
    sin = torch.cat([table[..., 1], table[..., 1]], -1)[:, None, :].to(x.dtype)
    rot = torch.cat([-x[..., hd // 2 :], x[..., : hd // 2]], -1)
    return x * cos + rot * sin


def _norm(cfg: DecoderConfig, w: dict, prefix: str, x: torch.Tensor) -> torch.Tensor:
    if cfg.norm == "rms":
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w[prefix + ".weight"]
    return F.layer_norm(x, (x.shape[-1],), w[prefix + ".weight"], w[prefix + ".bias"], cfg.norm_eps)


def decoder_hidden(cfg: DecoderConfig, w: dict[str, torch.Tensor], tok: torch.Tensor, rope_table=None, routing=None) -> torch.Tensor:
    """Final-norm hidden states ``[T, d]`` for one sequence. ``w`` maps slot names to (float) tensors. ``routing``
    (optional, list of ``[T, top_k]`` index tensors per layer) fixes the expert choice of MoE layers, which makes the
    function comparable with a lower-precision run whose near-tied router scores resolve differently."""
    T = tok.numel()
    H, KV, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    x = w["embed"][tok.long()]
    if cfg.pos == "learned":
        x = x + w["wpe"][:T]
    for li in range(cfg.n_layers):
        p = f"layers.{li}."
        xn = _norm(cfg, w, p + "norm1", x)
        qkv = xn @ w[p + "wqkv"].T
        if cfg.bias or cfg.qkv_bias:
            qkv = qkv + w[p + "bqkv"]
        qf, kf = qkv[:, : H * hd], qkv[:, H * hd : (H + KV) * hd]
        if cfg.qk_norm == "head":
            qh, kh = qf.reshape(T, H, hd), kf.reshape(T, KV, hd)
            qf = (qh * torch.rsqrt(qh.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w[p + "q_norm.weight"]).reshape(T, H * hd)
            kf = (kh * torch.rsqrt(kh.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w[p + "k_norm.weight"]).reshape(T, KV * hd)
        elif cfg.qk_norm:
            qf = qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w[p + "q_norm.weight"]
            kf = kf * torch.rsqrt(kf.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w[p + "k_norm.weight"]
        q = qf.reshape(T, H, hd)
        k = kf.reshape(T, KV, hd)
        v = qkv[:, (H + KV) * hd :].view(T, KV, hd)
        if cfg.pos == "rope":
            q, k = _rope(q, rope_table[:T]), _rope(k, rope_table[:T])
        rep = H // KV
        kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        att = torch.einsum("thd,shd->hts", q, kk) / hd**0.5
        mask = torch.ones(T, T, dtype=torch.bool, device=x.device).tril()
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        o = torch.einsum("hts,shd->thd", att, vv).reshape(T, H * hd)
        o = o @ w[p + "wo"].T
        if cfg.bias:
            o = o + w[p + "bo"]
        x = x + o
        xn2 = _norm(cfg, w, p + "norm2", x)
        if cfg.n_experts:
            probs = (xn2 @ w[p + "router"].T).float().softmax(-1)
            if routing is not None:
                topi = routing[li].long()
                topw = probs.gather(1, topi)
            else:
                topw, topi = torch.topk(probs, cfg.top_k, dim=-1)
            if cfg.norm_topk_prob:
                topw = topw / topw.sum(-1, keepdim=True)
            gate = torch.zeros_like(probs).scatter(1, topi, topw).to(x.dtype)          # [T, E], zero off the top-k
            gu = torch.einsum("td,efd->tef", xn2, w[p + "experts.wgu"])
            h = F.silu(gu[..., 0::2]) * gu[..., 1::2]
            y = torch.einsum("tei,edi->ted", h, w[p + "experts.wd"])
            x = x + (y * gate.unsqueeze(-1)).sum(1)
        elif cfg.act in ("swiglu", "geglu"):
            gu = xn2 @ w[p + "wgu"].T
            g, u = gu[:, 0::2], gu[:, 1::2]
            a = (F.silu(g) if cfg.act == "swiglu" else F.gelu(g, approximate="tanh")) * u
            x = x + a @ w[p + "wd"].T
        else:
            h = xn2 @ w[p + "wfc"].T
            if cfg.bias:
                h = h + w[p + "bfc"]
            h = F.gelu(h, approximate="tanh") @ w[p + "wproj"].T
            if cfg.bias:
                h = h + w[p + "bproj"]
            x = x + h
    return _norm(cfg, w, "norm_f", x)


def example_loss(cfg: DecoderConfig, w: dict[str, torch.Tensor], tok: torch.Tensor, labels: torch.Tensor,
                 rope_table=None, routing=None) -> torch.Tensor:
    """Mean NLL over the supervised positions of one sequence (labels already shifted; negative = ignored)."""
    h = decoder_hidden(cfg, w, tok, rope_table, routing)
    head = w["embed"] if cfg.tie_embeddings else w["lm_head"]
    logits = h @ head.T
    nll = F.cross_entropy(logits, labels.long().clamp(min=0), reduction="none")
    valid = (labels >= 0).to(nll.dtype)
    return (nll * valid).sum() / valid.sum().clamp(min=1.0)
