"""Mixture-of-experts MLP for the generic (``vmap``) path (packages/opake-patches/src/opake/api/patches/kernels/
moe.py:517,570-627, fused_moe.py:53-480, _moe_dispatch.py:106-195, _moe_memory.py).

``opake_moe(x, gate_up_proj, down_proj, top_k_index, top_k_weights)`` computes
``sum_k w[t,k] * down[e] (silu(gate[e] x_t) * up[e] x_t)`` for ``e = index[t,k]``. Two routes:

* ``grouped=True``: tokens are sorted by expert and each expert runs one GEMM pair on its contiguous slice (what the
  reference does with ``torch._grouped_mm``); on CUDA bf16 the per-expert products use the tcgen05 GEMM.
* ``grouped=False``: the dense baseline: every expert runs on every token and the result is masked. Exact, simple,
  E/k times more FLOPs; it is the oracle of the grouped route.

``moe_dispatch_plan`` chooses between them from a FLOP / memory estimate; ``per_example_expert_grad_sq_norms`` gives
per-example squared gradient norms of the expert weights for a batch of examples without a ``(B, E, ...)`` tensor, by
looping experts and using the Gram identity per (example, expert) group.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

__all__ = ["opake_moe", "dense_moe", "grouped_moe", "moe_dispatch_plan", "moe_memory_bytes", "per_example_expert_grad_sq_norms"]


def _act(g, u):
    return F.silu(g) * u


def dense_moe(x, gate_up_proj, down_proj, top_k_index, top_k_weights):
    """``x [T, d]``, ``gate_up_proj [E, 2I, d]`` (gate rows then up rows), ``down_proj [E, d, I]``."""
    E, I2, _ = gate_up_proj.shape
    I = I2 // 2
    T = x.shape[0]
    w = torch.zeros(T, E, dtype=x.dtype, device=x.device).scatter_add_(1, top_k_index, top_k_weights.to(x.dtype))
    gu = torch.einsum("td,efd->tef", x, gate_up_proj)
    h = _act(gu[..., :I], gu[..., I:])
    y = torch.einsum("tei,edi->ted", h, down_proj)
    return (y * w.unsqueeze(-1)).sum(1)


def grouped_moe(x, gate_up_proj, down_proj, top_k_index, top_k_weights):
    E, I2, d = gate_up_proj.shape
    I = I2 // 2
    T, k = top_k_index.shape
    flat_e = top_k_index.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // k
    counts = torch.bincount(flat_e, minlength=E)
    xs = x[tok]                                              # [T*k, d] sorted by expert
    ws = top_k_weights.reshape(-1)[order].to(x.dtype)
    out = torch.zeros_like(x)
    bounds = torch.cumsum(counts, 0).tolist()
    lo = 0
    pieces = []
    for e, hi in enumerate(bounds):
        if hi > lo:
            xe = xs[lo:hi]
            gu = xe @ gate_up_proj[e].t()
            pieces.append(_act(gu[:, :I], gu[:, I:]) @ down_proj[e].t())
        lo = hi
    ys = torch.cat(pieces, 0) if pieces else xs.new_zeros(0, d)
    out = out.index_add(0, tok, ys * ws.unsqueeze(-1))
    return out


def moe_memory_bytes(T: int, d: int, I: int, E: int, k: int, itemsize: int = 2) -> dict:
    """Activation bytes of one forward pass for the two routes."""
    return {"dense": T * E * (2 * I + I + d) * itemsize, "grouped": T * k * (d + 2 * I + I + d) * itemsize}


def moe_dispatch_plan(T: int, d: int, I: int, E: int, k: int, *, memory_budget: int | None = None) -> str:
    """``"grouped"`` unless the problem is so small that sorting costs more than the wasted FLOPs."""
    dense_flops = 6 * T * E * I * d
    grouped_flops = 6 * T * k * I * d
    if memory_budget is not None and moe_memory_bytes(T, d, I, E, k)["dense"] > memory_budget:
        return "grouped"
    return "dense" if (T * k < 4 * E and dense_flops < 64 * grouped_flops) else "grouped"


def opake_moe(x, gate_up_proj, down_proj, top_k_index, top_k_weights, *, grouped: bool = True):
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    idx, wts = top_k_index.reshape(x2.shape[0], -1), top_k_weights.reshape(x2.shape[0], -1)
    fn = grouped_moe if grouped and not torch._C._functorch.is_batchedtensor(x2) else dense_moe
    return fn(x2, gate_up_proj, down_proj, idx, wts).view(*lead, -1)


def per_example_expert_grad_sq_norms(x, dy_h, h, dy, example_id, top_k_index, n_examples: int):
    """Squared norms of the expert weight gradients per example.

    ``x [N, d]`` expert inputs, ``dy_h [N, 2I]`` gradients at the gate/up outputs, ``h [N, I]`` activations,
    ``dy [N, d]`` gradients at the expert outputs, all in (token, slot) order flattened to ``N = T * k`` rows;
    ``example_id [N]`` and ``top_k_index`` flattened ``[N]``. For each (example, expert) group the gradient of a
    weight is ``G^T X`` over the group's rows, whose squared norm is ``sum((G G^T) * (X X^T))``.
    """
    out = torch.zeros(n_examples, dtype=torch.float64, device=x.device)
    key = example_id.long() * (int(top_k_index.max().item()) + 1) + top_k_index.long()
    order = torch.argsort(key, stable=True)
    key_s = key[order]
    uniq, counts = torch.unique_consecutive(key_s, return_counts=True)
    lo = 0
    E1 = int(top_k_index.max().item()) + 1
    for u, c in zip(uniq.tolist(), counts.tolist()):
        rows = order[lo:lo + c]
        lo += c
        xe, ge, he, de = x[rows].float(), dy_h[rows].float(), h[rows].float(), dy[rows].float()
        n1 = ((ge @ ge.t()) * (xe @ xe.t())).sum()
        n2 = ((de @ de.t()) * (he @ he.t())).sum()
        out[u // E1] += (n1 + n2).double()
    return out
