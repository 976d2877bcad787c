"""Kernel-backed, vmap-safe operators used by the model patches (packages/opake-patches/src/opake/patches/kernels/
__init__.py). The ``opake_*`` names are the reference's public operator names; the shorter names are this package's."""
from ...ops.clip_sum import fused_clip_sum
from ...ops.lce import linear_cross_entropy, opake_linear_cross_entropy_loss
from .functions import (opake_cross_entropy, opake_fused_add_rms_norm, opake_geglu, opake_rms_norm, opake_rope_qk,
                        opake_selective_log_softmax, opake_swiglu)
from .lora import lora_grad_sq_norms, lora_linear, lora_mlp, lora_qkv
from .moe import dense_moe, grouped_moe, moe_dispatch_plan, opake_moe

# activation selectors of the fused LoRA MLP / gated-MLP operators
ACTIVATION_SWIGLU = "silu"
ACTIVATION_GEGLU_EXACT = "none"
ACTIVATION_GEGLU_APPROX = "tanh"


def opake_cross_entropy_loss(logits, labels, ignore_index: int = -100, logit_softcapping: float = 0.0, logit_scale: float = 1.0):
    """Per-token cross entropy (fp32, zero at ignored positions) of ``[..., V]`` logits against ``[...]`` labels."""
    return opake_cross_entropy(logits, labels, ignore_index=ignore_index, logit_scale=logit_scale, logit_softcapping=logit_softcapping)


def opake_geglu_exact(gate, up):
    return opake_geglu(gate, up, approximate="none")


def opake_geglu_approx(gate, up):
    return opake_geglu(gate, up, approximate="tanh")


def opake_rope(q, k, cos, sin, position_ids=None, unsqueeze_dim: int = 1):
    """Rotate-half rotary embedding of ``[B, H, T, hd]`` queries and keys: one kernel launch for both on CUDA bf16 when
    the tables do not depend on the batch index, the same formula in eager mode otherwise."""
    from ..transformers.components.rope import opake_apply_rotary_pos_emb

    return opake_apply_rotary_pos_emb(q, k, cos, sin, position_ids, unsqueeze_dim)


def opake_slow_rope(q, k, cos, sin, position_ids=None, unsqueeze_dim: int = 1):
    """The eager formula, always (per-example position ids, partial tables, CPU)."""
    from ..transformers.components.rope import _eager

    return _eager(q, k, cos, sin, unsqueeze_dim)


opake_lora_w = lora_linear
opake_lora_qkv = lora_qkv
opake_lora_mlp = lora_mlp

__all__ = ["fused_clip_sum", "linear_cross_entropy", "opake_linear_cross_entropy_loss", "opake_cross_entropy",
           "opake_cross_entropy_loss", "opake_fused_add_rms_norm", "opake_geglu", "opake_geglu_exact", "opake_geglu_approx",
           "opake_rms_norm", "opake_rope", "opake_rope_qk", "opake_slow_rope", "opake_selective_log_softmax", "opake_swiglu",
           "lora_linear", "lora_qkv", "lora_mlp", "lora_grad_sq_norms", "opake_lora_w", "opake_lora_qkv", "opake_lora_mlp",
           "opake_moe", "dense_moe", "grouped_moe", "moe_dispatch_plan", "ACTIVATION_SWIGLU", "ACTIVATION_GEGLU_EXACT",
           "ACTIVATION_GEGLU_APPROX"]
