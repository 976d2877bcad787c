"""vmap-safe building blocks that replace Hugging Face sub-module forwards (packages/opake-patches/src/opake/api/
patches/transformers/components/*.py). One module per concern: attention, normalisation / gated MLP, rotary
embedding, dropout, KV cache, batch-dimension shim, causal-LM loss (plain and fused with the LM head), expert blocks."""
from .attention import (SoftcappedAttention, causal_mask, eager_attention_forward, repeat_kv, sliding_window_mask, softcapped_attention,
                        softcapped_attention_recompute, vmap_sdpa_attention_forward)
from .batchify import apply_batchify_patch, batchify_forward
from .cross_entropy import (apply_causal_lm_loss_function_patch, apply_fused_linear_ce_patch, fused_linear_ce_supports,
                            make_fused_ce_causal_lm_forward, opake_causal_lm_loss)
from .dropout import disable_dropout
from .kv_cache import apply_kv_cache_patch, disable_kv_cache, disable_kv_cache_in_training
from .moe import dense_experts_forward
from .norm_mlp import patched_fused_gate_up_mlp_forward, patched_gated_mlp_forward, patched_rms_norm_forward
from .rope import apply_rope_patch, opake_apply_rotary_pos_emb

__all__ = ["SoftcappedAttention", "causal_mask", "eager_attention_forward", "repeat_kv", "sliding_window_mask", "softcapped_attention",
           "softcapped_attention_recompute", "vmap_sdpa_attention_forward", "apply_batchify_patch", "batchify_forward",
           "apply_causal_lm_loss_function_patch", "apply_fused_linear_ce_patch", "fused_linear_ce_supports",
           "make_fused_ce_causal_lm_forward", "opake_causal_lm_loss", "disable_dropout", "apply_kv_cache_patch", "disable_kv_cache",
           "disable_kv_cache_in_training", "dense_experts_forward", "patched_fused_gate_up_mlp_forward", "patched_gated_mlp_forward",
           "patched_rms_norm_forward", "apply_rope_patch", "opake_apply_rotary_pos_emb"]
