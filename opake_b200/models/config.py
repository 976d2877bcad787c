"""Decoder architecture descriptions and the named shapes used by the benchmarks."""
from __future__ import annotations

from dataclasses import dataclass, field, replace


@dataclass(frozen=True)
class DecoderConfig:
    name: str
    vocab_size: int
    d_model: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    max_seq: int = 2048
    norm: str = "rms"              # "rms" | "layer"
    norm_eps: float = 1e-5
    act: str = "swiglu"            # "swiglu" | "gelu" (GPT-2 two-matrix MLP) | "geglu"
    pos: str = "rope"              # "rope" | "learned"
    rope_theta: float = 500000.0
    rope_scaling: dict | None = None
    tie_embeddings: bool = False
    bias: bool = False             # GPT-2 style biases on every projection
    # mixture of experts (0 experts = dense MLP)
    n_experts: int = 0
    top_k: int = 0
    expert_ffn: int = 0
    norm_topk_prob: bool = False
    # RMSNorm of queries and keys before RoPE. True / "proj": over the whole projection (OLMoE, weight [H * hd]);
    # "head": per head over head_dim with one weight [hd] shared by all heads (Qwen3)
    qk_norm: bool | str = False
    # bias on the fused q/k/v projection only (Qwen2); ``bias`` puts one on every projection (GPT-2)
    qkv_bias: bool = False
    family: str = "llama"

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim

    def num_params(self) -> int:
        from .flat import build_layout

        return build_layout(self).total


def llama3_8b(**kw) -> DecoderConfig:
    return replace(DecoderConfig("llama3-8b", 128256, 4096, 32, 32, 8, 128, 14336, 2048), **kw)


def llama32_1b(**kw) -> DecoderConfig:
    return replace(DecoderConfig("llama3.2-1b", 128256, 2048, 16, 32, 8, 64, 8192, 2048, tie_embeddings=True), **kw)


def gpt2_small(**kw) -> DecoderConfig:
    return replace(DecoderConfig("gpt2-small", 50257, 768, 12, 12, 12, 64, 3072, 1024, norm="layer", act="gelu",
                                 pos="learned", tie_embeddings=True, bias=True, family="gpt2"), **kw)


def olmoe_1b_7b(**kw) -> DecoderConfig:
    return replace(DecoderConfig("olmoe-1b-7b", 50304, 2048, 16, 16, 16, 128, 0, 2048, rope_theta=10000.0, n_experts=64,
                                 top_k=8, expert_ffn=1024, qk_norm=True, family="olmoe"), **kw)


def tiny_llama(**kw) -> DecoderConfig:
    return replace(DecoderConfig("tiny-llama", 512, 256, 2, 4, 2, 64, 512, 128), **kw)


PRESETS = {
    "llama3-8b": llama3_8b, "llama3.2-1b": llama32_1b, "gpt2-small": gpt2_small, "olmoe-1b-7b": olmoe_1b_7b,
    "tiny-llama": tiny_llama,
}
