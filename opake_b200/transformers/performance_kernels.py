"""Maps the trainer's kernel switches onto ``opake_b200.patches`` (packages/opake-transformers/src/opake/api/
transformers/trainer/_performance_kernels.py:1-60). Keys of ``performance_kernels_config``: rope, rms_norm,
activation, cross_entropy, fused_linear_cross_entropy, chunked_linear_cross_entropy, kv_cache, eager_attention,
batchify. ``use_compat_patches`` selects the compatibility bucket, ``use_performance_kernels`` the kernel bucket; the
``performance`` bucket (kv-cache handling) is always on."""
from __future__ import annotations

__all__ = ["PERFORMANCE_KERNEL_KEYS", "apply_performance_kernels"]

PERFORMANCE_KERNEL_KEYS = ("rope", "rms_norm", "activation", "cross_entropy", "fused_linear_cross_entropy",
                           "chunked_linear_cross_entropy", "kv_cache", "eager_attention", "batchify")


def apply_performance_kernels(model, args):
    from .. import patches
    cfg = dict(args.performance_kernels_config or {})
    unknown = set(cfg) - set(PERFORMANCE_KERNEL_KEYS)
    if unknown:
        from ..base.exceptions import ConfigurationError
        raise ConfigurationError(f"unknown performance_kernels_config keys {sorted(unknown)}; known: {PERFORMANCE_KERNEL_KEYS}")
    return patches.apply_model_patches(model, performance=True, compat=bool(args.use_compat_patches), peft=True,
                                       kernels=bool(args.use_performance_kernels),
                                       fused_linear_cross_entropy=cfg.get("fused_linear_cross_entropy"), **{
                                           k: v for k, v in cfg.items() if k != "fused_linear_cross_entropy"})
