"""Expert-block replacements for mixture-of-experts decoders (packages/opake-patches/src/opake/api/patches/
transformers/components/moe.py; kernels in patches/kernels/moe.py).

``dense_experts_forward`` evaluates every expert on every token and masks by the routing weights: no data-dependent
shapes, so it is legal under ``vmap`` for any expert container that exposes stacked ``gate_up_proj`` / ``down_proj``
parameters (Hugging Face v5 ``*Experts`` modules). It is the fallback when the grouped path's gate refuses (CPU
under vmap); the native runtime uses grouped tcgen05 GEMMs instead."""
from __future__ import annotations

import torch

from ...kernels.functions import opake_swiglu

__all__ = ["dense_experts_forward"]


def dense_experts_forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor:
    """``hidden_states [T, D]``, ``top_k_index [T, k]``, ``top_k_weights [T, k]`` -> ``[T, D]``."""
    E = self.gate_up_proj.shape[0]
    w = torch.zeros(hidden_states.shape[0], E, dtype=top_k_weights.dtype, device=hidden_states.device)
    w = w.scatter_add(1, top_k_index.long(), top_k_weights)
    gu = torch.einsum("td,efd->tef", hidden_states, self.gate_up_proj)         # [T, E, 2I]
    g, u = gu.chunk(2, dim=-1)
    y = torch.einsum("tei,edi->ted", opake_swiglu(g, u), self.down_proj)       # [T, E, D]
    return (y * w[..., None].to(y.dtype)).sum(1)
