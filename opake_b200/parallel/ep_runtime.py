"""Expert-parallel training state of a mixture-of-experts decoder: every rank keeps ``E / world`` experts of every layer.

The dense part of the model (attention, norms, routers, embeddings) stays data parallel: replicated parameters, summed
clipped gradients. The expert matrices are sharded by expert over the ranks and never replicated: a rank holds the
parameters, the fp32 clipped-gradient sums and the optimizer moments of ITS experts only, in buffers of their own
(``params``, ``acc``, ``m``, ``v``: flat, layer by layer, ``wgu`` then ``wd``). Tokens travel to the experts' owners and
back inside ``FusedExpertParallelLayer`` (dispatch / combine kernels over peer memory, grouped tcgen05 GEMMs).

Per-example clipping across ranks (the two-pass protocol of ``expert_parallel.py``): the backward pass of a layer
returns, per SOURCE example, the squared norm of that example's gradient w.r.t. the local experts and stores no
expert gradient. After the whole backward the ranks sum these vectors together with each example's dense squared norm
(one small all-reduce), every rank derives the clip factor of every example, and pass 2 forms the clipped expert
gradient sums with the factors folded into the GEMM operand rows.

The reference trains mixture-of-experts models on one device only (packages/opake-patches/src/opake/api/patches/kernels/
moe.py:570-627, fused_moe.py:389-480, per-example expert gradients materialised through virtual expert ids).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import DecoderConfig
from ..ops import kernels as K
from .ep_fused import EpContext, FusedExpertParallelLayer

__all__ = ["ExpertParallelRuntime"]

_bf16 = torch.bfloat16


class ExpertParallelRuntime:
    def __init__(self, cfg: DecoderConfig, router_weights: list[torch.Tensor], tokens: int, device: torch.device, *,
                 init_seed: int = 0, std: float = 0.02, group=None):
        if not cfg.n_experts or cfg.act != "swiglu":
            raise ValueError("expert parallelism needs a mixture-of-experts decoder with SwiGLU experts")
        self.cfg, self.device, self.T = cfg, device, tokens
        self.ctx = EpContext(cfg.n_experts, tokens * cfg.top_k, device, group)
        self.world, self.rank = self.ctx.world, self.ctx.rank
        El, I, d, L = self.ctx.e_local, cfg.expert_ffn, cfg.d_model, cfg.n_layers
        self.n_wgu, self.n_wd = El * 2 * I * d, El * d * I
        self.per_layer = self.n_wgu + self.n_wd
        self.total = L * self.per_layer
        self.params = torch.empty(self.total, dtype=_bf16, device=device)
        self.acc = torch.zeros(self.total, dtype=torch.float32, device=device)
        self.m = torch.zeros(self.total, dtype=torch.float32, device=device)
        self.v = torch.zeros(self.total, dtype=torch.float32, device=device)
        self._init_params(init_seed, std)
        self.layers = []
        for li in range(L):
            wgu, wd = self.views(self.params, li)
            self.layers.append(FusedExpertParallelLayer(self.ctx, router_weights[li], wgu, wd, tokens, cfg.top_k,
                                                        cfg.norm_topk_prob))
        self.norms = torch.zeros(self.world, dtype=torch.float64, device=device)       # per source example
        self._norms_sum = torch.zeros(self.world, dtype=torch.float64, device=device)
        self.scales = torch.zeros(self.world, dtype=torch.float32, device=device)
        self._norm_parts: list[torch.Tensor] = []

    def views(self, buf: torch.Tensor, li: int):
        El, I, d = self.ctx.e_local, self.cfg.expert_ffn, self.cfg.d_model
        base = li * self.per_layer
        return (buf[base : base + self.n_wgu].view(El, 2 * I, d),
                buf[base + self.n_wgu : base + self.per_layer].view(El, d, I))

    def _init_params(self, seed: int, std: float) -> None:
        """Experts are drawn per GLOBAL expert id, so the model does not depend on how many ranks share it."""
        from ..models.decoder import init_expert_

        cfg, El = self.cfg, self.ctx.e_local
        for li in range(cfg.n_layers):
            wgu, wd = self.views(self.params, li)
            for j in range(El):
                init_expert_(wgu[j], wd[j], seed, li, self.rank * El + j, cfg.n_layers, std)

    # ------------------------------------------------------------------ per example
    def begin_example(self) -> None:
        self._norm_parts.clear()
        self.ctx.begin_sequence()

    def end_example(self) -> None:
        self.ctx.end_sequence()

    def forward(self, li: int, x: torch.Tensor, residual: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        return self.layers[li].forward(x, residual=residual, out=out)

    def backward(self, li: int, dy: torch.Tensor, *, router_grad_out: torch.Tensor, sumsq: torch.Tensor, dx_out: torch.Tensor):
        dx, _, norms = self.layers[li].backward(dy, router_grad_out=router_grad_out, sumsq=sumsq, dx_out=dx_out)
        self._norm_parts.append(norms)
        return dx

    def clip_factors(self, dense_sumsq: torch.Tensor, clip: float, *, auto: bool = False, gamma: float = 0.01, n_leaves: int = 1,
                     widest_leaf: int = 1, counters: torch.Tensor | None = None) -> torch.Tensor:
        """Squared gradient norm of EVERY rank's current example (dense part on its home rank plus the expert parts
        on the experts' owners, one all-reduce of ``world`` doubles) and from it every example's guarded clip factor
        (float32 ``[world]``, the same on all ranks). ``dense_sumsq`` is this rank's example's dense squared norm."""
        self.norms.zero_()
        for part in self._norm_parts:
            self.norms.add_(part)
        self.norms[self.rank : self.rank + 1].add_(dense_sumsq.reshape(1))
        if self.world > 1:
            self.ctx.allreduce_f64(self.norms, self._norms_sum)
            self.norms.copy_(self._norms_sum)
        for r in range(self.world):
            K.clip_scale(self.norms[r : r + 1], clip, scale_out=self.scales[r : r + 1], auto=auto, gamma=gamma, n_leaves=n_leaves,
                         widest_leaf=widest_leaf, counters=counters if r == self.rank else None, reset=False)
        return self.scales

    def accumulate_clipped(self) -> None:
        """Pass 2: ``acc += sum_b scale_b * dW_experts^(b)`` for every layer's local experts."""
        for li, layer in enumerate(self.layers):
            acc_wgu, acc_wd = self.views(self.acc, li)
            layer.accumulate_clipped(self.scales, acc_wgu, acc_wd)

    # ------------------------------------------------------------------ optimizer step
    def apply_update(self, *, noise_offset: int, inv_batch: float, sigma: float, seed: int, step: int, lr: float, beta1: float,
                     beta2: float, eps: float, weight_decay: float, bc1: float, bc2: float, phi_hat: float, sgd_mode: bool) -> None:
        """Noise and optimizer step on this rank's experts. No reduction across ranks: the owner already holds the sum
        over all examples. ``noise_offset`` places the experts in the global Philox index space behind the dense
        parameters and behind the lower ranks' experts, so every expert element draws its own noise exactly once."""
        begin = noise_offset + self.rank * self.total
        K.dp_step(grad_src=[self.acc.data_ptr() - 4 * begin], shard_begin=begin, shard_len=self.total, inv_batch=inv_batch,
                  sigma=sigma, seed=seed, step=step, m=self.m, v=self.v, master=None,
                  param_dst=[self.params.data_ptr() - 2 * begin], param_src=_Shifted(self.params, begin), lr=lr, beta1=beta1,
                  beta2=beta2, eps=eps, weight_decay=weight_decay, bc1=bc1, bc2=bc2, phi_hat=phi_hat, zero_grad=True,
                  sgd_mode=sgd_mode, device=self.device)

    def state_dict(self) -> dict:
        return {"rank": self.rank, "world": self.world, "params": self.params.cpu(), "m": self.m.cpu(), "v": self.v.cpu()}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank:
            raise ValueError("expert-parallel checkpoint was written for another rank layout")
        self.params.copy_(sd["params"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])


class _Shifted:
    """Stand-in for a tensor whose element 0 sits ``begin`` elements before the real buffer (the fused step addresses
    its parameter source with global element offsets)."""

    def __init__(self, t: torch.Tensor, begin: int):
        self._ptr = t.data_ptr() - t.element_size() * begin

    def data_ptr(self) -> int:
        return self._ptr
