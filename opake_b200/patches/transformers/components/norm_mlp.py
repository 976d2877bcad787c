"""Forward replacements for normalisation and gated-MLP modules (packages/opake-patches/src/opake/api/patches/
transformers/components/rms_norm.py, fused_add_rms_norm.py, and the activation swaps of _factory.py:186): the module's
own parameters, this package's vmap-safe kernel functions."""
from __future__ import annotations

from ...kernels.functions import opake_geglu, opake_rms_norm, opake_swiglu

__all__ = ["patched_rms_norm_forward", "patched_gated_mlp_forward", "patched_fused_gate_up_mlp_forward"]


def patched_rms_norm_forward(self, hidden_states):
    """Forward for ``*RMSNorm`` modules: fused kernel on CUDA bf16, same formula elsewhere. Modules that store
    ``weight - 1`` (Gemma) are recognised by ``_opake_offset``."""
    eps = getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6))
    return opake_rms_norm(hidden_states, self.weight, eps, getattr(self, "_opake_offset", 0.0))


def patched_gated_mlp_forward(self, x):
    act = getattr(self, "_opake_act", "silu")
    g, u = self.gate_proj(x), self.up_proj(x)
    return self.down_proj(opake_swiglu(g, u) if act == "silu" else opake_geglu(g, u, approximate=act))


def patched_fused_gate_up_mlp_forward(self, x):
    """Phi-3 / GLM-4 layout: one ``gate_up_proj`` whose output is ``[gate | up]`` along the last axis."""
    act = getattr(self, "_opake_act", "silu")
    g, u = self.gate_up_proj(x).chunk(2, dim=-1)
    return self.down_proj(opake_swiglu(g, u) if act == "silu" else opake_geglu(g, u, approximate=act))
