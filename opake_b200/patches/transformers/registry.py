"""Model-family registry (packages/opake-patches/src/opake/api/patches/transformers/models/__init__.py:16-41,
_family.py:121-246, _factory.py:186, _registry.py). Each family names the module classes to patch (by class-name
suffix, so no Hugging Face import is needed to register), the activation of its gated MLP, whether its RMSNorm stores
``weight - 1``, attention extras, and whether the decoder can be lowered to the native flat-parameter runtime."""
from __future__ import annotations

from dataclasses import dataclass

__all__ = ["FamilySpec", "FAMILIES", "family_of", "register_family"]


@dataclass(frozen=True)
class FamilySpec:
    model_type: str
    norm_suffixes: tuple = ("RMSNorm",)
    mlp_suffixes: tuple = ("MLP",)
    act: str = "silu"                 # "silu" | "tanh" (gelu_pytorch_tanh) | "none" (exact gelu)
    norm_offset: float = 0.0          # 1.0: weights are stored minus one (Gemma)
    softcap: float | None = None      # attention logit soft-capping
    sliding_window: bool = False
    moe: bool = False
    native: bool = False              # lowers to DecoderConfig / NativeCausalLM
    rope: bool = True                 # rotate-half ``apply_rotary_pos_emb`` in the modeling module (replaced by the kernel)
    fused_gate_up: bool = False       # MLP stores one ``gate_up_proj`` ([gate | up]) instead of two projections
    notes: str = ""


FAMILIES: dict[str, FamilySpec] = {}


def register_family(spec: FamilySpec) -> FamilySpec:
    FAMILIES[spec.model_type] = spec
    return spec


for _s in (
    FamilySpec("llama", native=True), FamilySpec("mistral", sliding_window=True, native=True), FamilySpec("ministral", sliding_window=True),
    FamilySpec("mellum", native=True), FamilySpec("smollm3", native=True), FamilySpec("granite", notes="residual / logit multipliers"),
    FamilySpec("qwen2", native=True, notes="q/k/v bias"), FamilySpec("qwen3", native=True, notes="per-head q/k norm"), FamilySpec("olmo2", notes="post-norm, q/k norm"),
    FamilySpec("olmo3", sliding_window=True, notes="post-norm, q/k norm"), FamilySpec("phi3", fused_gate_up=True, notes="fused qkv and gate_up"),
    FamilySpec("glm4", fused_gate_up=True, rope=False, notes="fused gate_up, extra norms, interleaved partial rotary"), FamilySpec("exaone4", sliding_window=True, notes="q/k norm"),
    # Cohere's "LayerNorm" subtracts the mean: it is not an RMSNorm and keeps its stock forward
    FamilySpec("cohere", norm_suffixes=(), rope=False, notes="parallel block, bias-free mean-subtracting layer norm"),
    FamilySpec("cohere2", norm_suffixes=(), sliding_window=True, rope=False),
    FamilySpec("gemma", act="tanh", norm_offset=1.0), FamilySpec("gemma2", act="tanh", norm_offset=1.0, softcap=50.0, sliding_window=True),
    FamilySpec("gemma3", act="tanh", norm_offset=1.0, sliding_window=True, notes="q/k norm, local/global rope"),
    FamilySpec("gemma3_text", act="tanh", norm_offset=1.0, sliding_window=True, notes="text tower of gemma3"),
    FamilySpec("gpt2", norm_suffixes=(), mlp_suffixes=(), act="none", native=True, rope=False, notes="LayerNorm, learned positions, Conv1D"),
    FamilySpec("gpt_oss", moe=True, sliding_window=True, notes="attention sinks, clamped swiglu"),
    FamilySpec("mixtral", moe=True, sliding_window=True), FamilySpec("qwen3_moe", moe=True), FamilySpec("qwen3_5_moe", moe=True),
    FamilySpec("qwen3_next", moe=True, notes="gated delta-net layers stay on the stock path"),
    FamilySpec("hunyuan_v1_moe", moe=True), FamilySpec("deepseek_v4", moe=True, rope=False, notes="MLA attention stays on the stock path"),
    FamilySpec("olmoe", moe=True, native=True, notes="not patched by the reference; native MoE runtime target"),
):
    register_family(_s)


def family_of(model) -> FamilySpec | None:
    cfg = getattr(model, "config", None)
    mt = getattr(cfg, "model_type", None) or getattr(cfg, "family", None)
    return FAMILIES.get(mt)
