"""Flat parameter layout.

All parameters of a decoder live in ONE contiguous bf16 buffer (and the per-example gradient, the fp32
clipped-gradient accumulator and the optimizer moments in buffers with the same element order). A flat order makes
the sharded optimizer trivial (rank r owns ``[r*S, (r+1)*S)``), lets the Philox noise be indexed by the global
element offset, and turns the clip-accumulate and the fused step into single launches.

Order: every dense tensor first (layers, final norm, LM head, position table), the token-embedding table last,
because its per-example gradient is sparse and handled row-wise.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .config import DecoderConfig

ALIGN = 128  # elements; keeps every view 256-byte aligned for TMA and vector access


@dataclass(frozen=True)
class Slot:
    name: str
    shape: tuple[int, ...]
    offset: int

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass(frozen=True)
class Layout:
    slots: tuple[Slot, ...]
    total: int        # padded element count of the whole buffer
    dense_total: int  # elements before the (sparse-gradient) token embedding
    n_params: int     # true parameter count (no padding)

    def slot(self, name: str) -> Slot:
        for s in self.slots:
            if s.name == name:
                return s
        raise KeyError(name)

    def shard_bounds(self, world: int) -> list[int]:
        """``world + 1`` offsets cutting the flat vector into contiguous shards of nearly equal size whose boundaries
        fall on tensor boundaries, so every tensor has exactly one owner: a weight matrix can then be fetched from its
        owner by one GEMM, and the embedding rows are accumulated on one rank. Offsets are multiples of ``ALIGN``.
        A model with fewer tensors than ranks leaves some shards empty."""
        cuts = sorted({s.offset for s in self.slots} | {self.total})
        bounds = [0]
        for r in range(1, world):
            target = self.total * r / world
            cand = [c for c in cuts if c >= bounds[-1]]
            bounds.append(min(cand, key=lambda c: abs(c - target)))
        bounds.append(self.total)
        return bounds

    def owner_of(self, name: str, bounds: list[int]) -> int:
        off = self.slot(name).offset
        for r in range(len(bounds) - 1):
            if bounds[r] <= off < bounds[r + 1]:
                return r
        raise KeyError(name)

    def views(self, buf: torch.Tensor, dense_only: bool = False) -> dict[str, torch.Tensor]:
        out = {}
        for s in self.slots:
            if dense_only and s.offset >= self.dense_total:
                continue
            out[s.name] = buf[s.offset : s.offset + s.numel].view(s.shape)
        return out


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


def build_layout(cfg: DecoderConfig, shard_multiple: int = 1, skip_experts: bool = False) -> Layout:
    """``skip_experts``: leave the expert matrices of mixture-of-experts layers out (expert parallelism keeps every
    rank's experts in a separate, rank-private buffer; the router stays here)."""
    slots: list[Slot] = []
    off = 0
    n_params = 0

    def add(name: str, *shape: int) -> None:
        nonlocal off, n_params
        s = Slot(name, tuple(shape), off)
        slots.append(s)
        n_params += s.numel
        off = _round_up(off + s.numel, ALIGN)

    d = cfg.d_model
    for i in range(cfg.n_layers):
        p = f"layers.{i}."
        add(p + "norm1.weight", d)
        if cfg.norm == "layer":
            add(p + "norm1.bias", d)
        add(p + "wqkv", cfg.qkv_dim, d)
        if cfg.bias or cfg.qkv_bias:
            add(p + "bqkv", cfg.qkv_dim)
        if cfg.qk_norm == "head":
            add(p + "q_norm.weight", cfg.head_dim)
            add(p + "k_norm.weight", cfg.head_dim)
        elif cfg.qk_norm:
            add(p + "q_norm.weight", cfg.n_heads * cfg.head_dim)
            add(p + "k_norm.weight", cfg.n_kv_heads * cfg.head_dim)
        add(p + "wo", d, cfg.n_heads * cfg.head_dim)
        if cfg.bias:
            add(p + "bo", d)
        add(p + "norm2.weight", d)
        if cfg.norm == "layer":
            add(p + "norm2.bias", d)
        if cfg.n_experts:
            add(p + "router", cfg.n_experts, d)
            if not skip_experts:
                add(p + "experts.wgu", cfg.n_experts, 2 * cfg.expert_ffn, d)
                add(p + "experts.wd", cfg.n_experts, d, cfg.expert_ffn)
        elif cfg.act in ("swiglu", "geglu"):
            add(p + "wgu", 2 * cfg.ffn, d)   # rows interleaved: 2j = gate_j, 2j+1 = up_j
            add(p + "wd", d, cfg.ffn)
        else:
            add(p + "wfc", cfg.ffn, d)
            if cfg.bias:
                add(p + "bfc", cfg.ffn)
            add(p + "wproj", d, cfg.ffn)
            if cfg.bias:
                add(p + "bproj", d)
    add("norm_f.weight", d)
    if cfg.norm == "layer":
        add("norm_f.bias", d)
    if cfg.pos == "learned":
        add("wpe", cfg.max_seq, d)
    if not cfg.tie_embeddings:
        add("lm_head", cfg.vocab_size, d)
        dense_total = off
        add("embed", cfg.vocab_size, d)
    else:
        # tied: the shared matrix receives a dense LM-head gradient, so it belongs to the dense region
        add("embed", cfg.vocab_size, d)
        dense_total = off
    total = _round_up(off, ALIGN * max(1, shard_multiple))
    return Layout(tuple(slots), total, dense_total, n_params)
