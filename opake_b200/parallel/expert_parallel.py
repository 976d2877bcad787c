"""Expert parallelism with per-example clipping: protocol layer.

Experts of a MoE layer are sharded over the ranks of a group (``E / world`` experts each). Every rank works on its own
example; tokens travel to the ranks that own their experts and back (two all-to-alls forward, two backward). The
difficulty that differential privacy adds: the owner of an expert sees rows of ``world`` DIFFERENT examples in one
batch of tokens, and each example must be clipped by ITS OWN gradient norm, which also contains the dense layers'
part that lives on the example's home rank. Materialising ``(world, E_local, ...)`` per-example expert gradients would
multiply memory by the group size; instead the backward runs in two passes over the token rows:

1. ``backward(dy)``: input gradients flow back as usual. For the expert weights only the per-(source example) squared
   gradient norms are computed, with the Gram identity ``||G^T X||_F^2 = sum((G G^T) * (X X^T))`` per (example,
   expert) group of rows, and returned as a ``[world]`` vector; nothing gradient-sized is stored.
2. the caller adds these to the dense squared norms of each example (an all-reduce of a ``[world]`` vector), derives
   the clip factors, and calls ``accumulate_clipped(scales)``: the weight-gradient products are formed ONCE over all
   rows with each row of the upstream gradient multiplied by the clip factor of the example it belongs to (the scale
   is folded into the GEMM operand), and added to the fp32 sums. This equals ``sum_b s_b * dW^(b)`` exactly.

The collectives here are ``torch.distributed.all_to_all_single`` (NCCL on GPUs, gloo on CPU ranks for the tests); the
single-GPU native runtime (``models/decoder.py``) uses the grouped tcgen05 GEMM modes for the same math.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

__all__ = ["ExpertParallelLayer", "route"]


def route(x: torch.Tensor, router_w: torch.Tensor, top_k: int, norm_topk: bool):
    probs = (x @ router_w.t()).to(torch.promote_types(x.dtype, torch.float32)).softmax(-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True)
    return probs, w, idx


def _a2a(t: torch.Tensor, in_split: list[int], out_split: list[int], group) -> torch.Tensor:
    out = t.new_empty((sum(out_split), *t.shape[1:]))
    dist.all_to_all_single(out, t.contiguous(), output_split_sizes=out_split, input_split_sizes=in_split, group=group)
    return out


@dataclass
class _Ctx:
    x: torch.Tensor
    probs: torch.Tensor
    w: torch.Tensor
    idx: torch.Tensor
    order: torch.Tensor           # entries sorted by destination rank (stable)
    send_counts: list[int]
    recv_counts: list[int]
    recv_x: torch.Tensor          # rows received from all ranks
    recv_e: torch.Tensor          # local expert id of every received row
    recv_src: torch.Tensor        # source rank (= example) of every received row
    gu: torch.Tensor
    h: torch.Tensor
    y_rows: torch.Tensor          # expert outputs returned to this rank, in entry order
    dy_rows: torch.Tensor | None = None
    dgu: torch.Tensor | None = None


class ExpertParallelLayer:
    """Expert-parallel SwiGLU MoE layer for one example per rank. ``wgu`` ``[E_local, 2I, d]`` (gate rows then up rows),
    ``wd`` ``[E_local, d, I]``; the router is replicated."""

    def __init__(self, router_w, wgu_local, wd_local, top_k: int, norm_topk: bool = False, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.router_w, self.wgu, self.wd = router_w, wgu_local, wd_local
        self.e_local = wgu_local.shape[0]
        self.top_k, self.norm_topk = top_k, norm_topk
        self.ctx: _Ctx | None = None

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T, d = x.shape
        k, W, El = self.top_k, self.world, self.e_local
        probs, w, idx = route(x, self.router_w, k, self.norm_topk)
        flat_e = idx.reshape(-1)
        dst_rank = flat_e // El
        order = torch.argsort(dst_rank, stable=True)
        send_counts = torch.bincount(dst_rank, minlength=W).tolist()
        if W > 1:
            counts_t = torch.tensor(send_counts, dtype=torch.int64, device=x.device)
            recv_t = torch.empty_like(counts_t)
            dist.all_to_all_single(recv_t, counts_t, group=self.group)
            recv_counts = recv_t.tolist()
        else:
            recv_counts = list(send_counts)
        tok = order // k
        send_x = x[tok]
        send_e = (flat_e[order] % El).to(torch.int64)
        if W > 1:
            recv_x = _a2a(send_x, send_counts, recv_counts, self.group)
            recv_e = _a2a(send_e, send_counts, recv_counts, self.group)
        else:
            recv_x, recv_e = send_x, send_e
        recv_src = torch.repeat_interleave(torch.arange(W, device=x.device), torch.tensor(recv_counts, device=x.device))
        I = self.wd.shape[-1]
        gu = torch.einsum("nd,nfd->nf", recv_x, self.wgu[recv_e]) if recv_x.shape[0] else recv_x.new_zeros(0, 2 * I)
        h = F.silu(gu[:, :I]) * gu[:, I:]
        y = torch.einsum("ni,ndi->nd", h, self.wd[recv_e]) if h.shape[0] else recv_x.new_zeros(0, d)
        back = _a2a(y, recv_counts, send_counts, self.group) if W > 1 else y
        y_rows = torch.empty_like(back)
        y_rows[order] = back                                   # entry order (t * k + slot)
        out = (y_rows.view(T, k, d) * w.to(x.dtype).unsqueeze(-1)).sum(1)
        self.ctx = _Ctx(x, probs, w, idx, order, send_counts, recv_counts, recv_x, recv_e, recv_src, gu, h, y_rows)
        return out

    # ------------------------------------------------------------------ backward, pass 1
    def backward(self, dy: torch.Tensor):
        """Returns ``(dx, d_router, expert_sq_norms)``: the input gradient and the router weight gradient of THIS
        rank's example, and the squared norms of the local experts' weight gradients for every source example."""
        c = self.ctx
        T, d = c.x.shape
        k, W = self.top_k, self.world
        I = self.wd.shape[-1]
        # through the weighted combination
        dw = (dy.unsqueeze(1) * c.y_rows.view(T, k, d)).sum(-1).to(c.probs.dtype)            # [T, k]
        d_rows = (dy.unsqueeze(1) * c.w.to(dy.dtype).unsqueeze(-1)).reshape(T * k, d)       # entry order
        send = d_rows[c.order]
        dy_rows = _a2a(send, c.send_counts, c.recv_counts, self.group) if W > 1 else send
        # expert backward on the owner
        dh = torch.einsum("nd,ndi->ni", dy_rows, self.wd[c.recv_e]) if dy_rows.shape[0] else dy_rows.new_zeros(0, I)
        g, u = c.gu[:, :I], c.gu[:, I:]
        sg = torch.sigmoid(g)
        dgu = torch.cat([dh * u * sg * (1 + g * (1 - sg)), dh * F.silu(g)], dim=1)
        dxs = torch.einsum("nf,nfd->nd", dgu, self.wgu[c.recv_e]) if dgu.shape[0] else c.recv_x.new_zeros(0, d)
        c.dy_rows, c.dgu = dy_rows, dgu
        # per-(source example) squared norms of the expert weight gradients, no gradient-sized tensor
        norms = torch.zeros(W, dtype=torch.float64, device=dy.device)
        key = c.recv_src * self.e_local + c.recv_e
        for kv in torch.unique(key).tolist():
            rows = (key == kv).nonzero().squeeze(1)
            X, H, Gd, Gu = c.recv_x[rows].double(), c.h[rows].double(), dy_rows[rows].double(), dgu[rows].double()
            norms[kv // self.e_local] += ((Gd @ Gd.t()) * (H @ H.t())).sum() + ((Gu @ Gu.t()) * (X @ X.t())).sum()
        # input gradients return to the home ranks
        back = _a2a(dxs, c.recv_counts, c.send_counts, self.group) if W > 1 else dxs
        dx_rows = torch.empty_like(back)
        dx_rows[c.order] = back
        dx = dx_rows.view(T, k, d).sum(1)
        # router (replicated weight, this rank's example only)
        probs = c.probs
        gsel = torch.zeros_like(probs)
        if self.norm_topk:
            sel = probs.gather(1, c.idx)
            S = sel.sum(-1, keepdim=True)
            dot = (dw * sel / S).sum(-1, keepdim=True)
            gsel.scatter_(1, c.idx, (dw - dot) / S)
        else:
            gsel.scatter_(1, c.idx, dw)
        dlogits = probs * (gsel - (probs * gsel).sum(-1, keepdim=True))
        d_router = dlogits.t().to(c.x.dtype) @ c.x
        dx = dx + dlogits.to(c.x.dtype) @ self.router_w
        return dx, d_router, norms

    # ------------------------------------------------------------------ backward, pass 2
    def accumulate_clipped(self, scales: torch.Tensor, acc_wgu: torch.Tensor, acc_wd: torch.Tensor) -> None:
        """``acc += sum_b scales[b] * dW^(b)`` for the local experts; ``scales`` is indexed by source rank."""
        c = self.ctx
        s = scales.to(c.dy_rows.dtype)[c.recv_src].unsqueeze(1)
        dys, dgus = c.dy_rows * s, c.dgu * s                    # clip factor folded into the GEMM operand rows
        for e in range(self.e_local):
            rows = (c.recv_e == e).nonzero().squeeze(1)
            if rows.numel():
                acc_wd[e] += (dys[rows].t() @ c.h[rows]).to(acc_wd.dtype)
                acc_wgu[e] += (dgus[rows].t() @ c.recv_x[rows]).to(acc_wgu.dtype)
