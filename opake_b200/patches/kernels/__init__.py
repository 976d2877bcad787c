"""Kernel-backed, vmap-safe operators used by the model patches."""
from ...ops.clip_sum import fused_clip_sum
from ...ops.lce import linear_cross_entropy, opake_linear_cross_entropy_loss
from .functions import (opake_cross_entropy, opake_fused_add_rms_norm, opake_geglu, opake_rms_norm, opake_rope_qk,
                        opake_selective_log_softmax, opake_swiglu)
from .lora import lora_grad_sq_norms, lora_linear, lora_mlp, lora_qkv
from .moe import dense_moe, grouped_moe, moe_dispatch_plan, opake_moe

__all__ = ["fused_clip_sum", "linear_cross_entropy", "opake_linear_cross_entropy_loss", "opake_cross_entropy",
           "opake_fused_add_rms_norm", "opake_geglu", "opake_rms_norm", "opake_rope_qk", "opake_selective_log_softmax",
           "opake_swiglu", "lora_linear", "lora_qkv", "lora_mlp", "lora_grad_sq_norms", "opake_moe", "dense_moe",
           "grouped_moe", "moe_dispatch_plan"]
