"""Expert parallelism on the native kernels: dispatch and combine are single kernels over peer memory.

Same protocol and the same two-pass per-example clipping as :mod:`opake_b200.parallel.expert_parallel` (which runs on
``torch.distributed`` all-to-alls and is the CPU-testable specification), but:

* the routing histogram exchange, the permutation by expert and the transfer of the rows are device kernels that
  store / load over NVLink (``csrc/kernels/ep.cu``); no split size ever reaches the host, so a layer is a fixed
  sequence of launches with static shapes,
* the expert products are the grouped modes of the tcgen05 GEMM (``tile_group`` for forward / input gradients,
  ``group_k`` for weight gradients), with SwiGLU and its backward fused into the epilogues,
* the per-(source example) squared norms of the expert weight gradients are the ``sum(C^2)`` epilogue of the grouped
  weight-gradient GEMM run with one batch entry per (local expert, source rank) group and no output (the layout pads
  every such group to whole 64-row reduction blocks), so nothing gradient-sized per example is ever stored.

One example per rank and per call, as in the protocol layer. ``wgu`` holds gate and up rows INTERLEAVED
(row ``2j`` = gate ``j``, row ``2j+1`` = up ``j``), the layout the SwiGLU epilogue consumes.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as G
from ..ops._protos import EpGroup, EpPeers
from . import comm

__all__ = ["EpContext", "FusedExpertParallelLayer"]

PHASE_COUNTS, PHASE_ROWS, PHASE_OUT, PHASE_DROWS, PHASE_DOUT, PHASE_BARRIER = range(6)
_bf16 = torch.bfloat16


def _L():
    return _lib.lib()


def _p(t):
    return None if t is None else t.data_ptr()


class EpContext:
    """Group state shared by all expert-parallel layers of a model: ranks, control blocks, epoch counters."""

    def __init__(self, n_experts: int, n_entries: int, device: torch.device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts % self.world or self.world > 8:
            raise ValueError(f"{n_experts} experts cannot be sharded over {self.world} ranks (at most 8)")
        self.device, self.n_experts, self.n_entries = device, n_experts, n_entries
        self.e_local = n_experts // self.world
        self.r_cap = _L().opk_ep_rows_capacity(self.world, n_entries, n_experts)
        self.ctrl = comm.alloc_peer_buffer(_L().opk_ep_ctrl_ints(self.world, n_experts), torch.int32, device, group)
        self.ctrl.local.zero_()
        if self.world > 1:                 # every control block is zero before anyone raises a flag in it
            torch.cuda.synchronize(device)
            dist.barrier(group)
        # Epoch numbers handed to the kernels are RELATIVE to two counters in device memory (exchange epochs, barrier
        # epochs): ``end_sequence`` adds what a sequence of calls consumed, on the stream. A captured CUDA graph of one
        # example therefore replays with fresh absolute epochs although its kernel arguments are frozen.
        self.epoch_dev = torch.zeros(2, dtype=torch.int32, device=device)
        self.g = EpGroup(self.world, self.rank, n_experts, self.r_cap, (ctypes.c_void_p * 8)(*self.ctrl.ptrs),
                         self.epoch_dev.data_ptr())
        self.epoch = 0
        self.barrier_epoch = 0
        self.err = _lib.err_word(device)
        # slots of the small fp64 all-reduce (per-example norms): [world][64] doubles on every rank
        self._sum_slots = comm.alloc_peer_buffer(8 * 64, torch.float64, device, group)
        self._sum_slots.local.zero_()
        self._sum_peers = EpPeers((ctypes.c_void_p * 8)(*self._sum_slots.ptrs))
        if self.world > 1:
            torch.cuda.synchronize(device)
            dist.barrier(group)

    def begin_sequence(self) -> None:
        """Start of a launch sequence that every rank issues identically (one example): relative epochs restart."""
        self.epoch = 0
        self.barrier_epoch = 0

    def end_sequence(self) -> None:
        """Moves the device-side epoch bases past the epochs this sequence used (stream-ordered)."""
        _lib.check(_L().opk_ep_advance(self.epoch_dev.data_ptr(), self.epoch, self.barrier_epoch, self._s()), "ep_advance")
        self.epoch = 0
        self.barrier_epoch = 0

    def allreduce_f64(self, local: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``out = sum over ranks of local`` for a float64 vector of at most 64 entries, on the exchange kernels (plain
        peer stores, bounded wait; capturable, no library collective)."""
        if local.dtype != torch.float64 or out.dtype != torch.float64 or local.numel() > 64 or out.numel() != local.numel():
            raise ValueError("allreduce_f64 takes float64 vectors of at most 64 entries")
        self.epoch += 1
        _lib.check(_L().opk_ep_allreduce_f64(self.g, self._sum_peers, _p(local), local.numel(), self.epoch, _p(out), _p(self.err),
                                             self._s()), "ep_allreduce_f64")
        return out

    def rows(self, width: int) -> tuple[torch.Tensor, EpPeers]:
        """A ``[r_cap, width]`` bf16 row buffer that every rank of the group can address."""
        pb = comm.alloc_peer_buffer(self.r_cap * width, _bf16, self.device, self.group)
        pb.local.zero_()
        peers = EpPeers((ctypes.c_void_p * 8)(*pb.ptrs))
        peers._keep = pb
        return pb.local.view(self.r_cap, width), peers

    def _s(self):
        return _lib.stream_ptr(self.device)

    def barrier(self) -> None:
        """Stream-ordered group barrier (flag stores to all peers, bounded wait for all peers' flags)."""
        self.barrier_epoch += 1
        _lib.check(_L().opk_ep_signal(self.g, PHASE_BARRIER, self.barrier_epoch, self._s()), "ep_signal")
        _lib.check(_L().opk_ep_wait(self.g, PHASE_BARRIER, self.barrier_epoch, _p(self.err), self._s()), "ep_wait")


class FusedExpertParallelLayer:
    """Expert-parallel SwiGLU MoE layer for one example per rank on the native kernels.

    ``router_w [E, d]`` replicated; ``wgu_local [E_local, 2I, d]`` (gate / up rows interleaved) and
    ``wd_local [E_local, d, I]`` are this rank's experts. All bf16 CUDA tensors.
    """

    def __init__(self, ctx: EpContext, router_w, wgu_local, wd_local, tokens: int, top_k: int, norm_topk: bool = False):
        self.ctx, self.T, self.k, self.norm_topk = ctx, tokens, top_k, norm_topk
        self.router_w, self.wgu, self.wd = router_w, wgu_local, wd_local
        E, d = router_w.shape
        El, I = wd_local.shape[0], wd_local.shape[-1]
        if E != ctx.n_experts or El != ctx.e_local or tokens * top_k != ctx.n_entries or wgu_local.shape != (El, 2 * I, d):
            raise ValueError("weights do not match the expert-parallel context")
        self.d, self.I, self.E, self.El = d, I, E, El
        dev, R, n = ctx.device, ctx.r_cap, ctx.n_entries
        i32 = dict(dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.recv_x, self.recv_x_peers = ctx.rows(d)
        self.ye, self.ye_peers = ctx.rows(d)
        self.dy_rows, self.dy_peers = ctx.rows(d)
        self.dxs, self.dxs_peers = ctx.rows(d)
        e = lambda *s: torch.zeros(*s, dtype=_bf16, device=dev)
        self.gu, self.act, self.dgu = e(R, 2 * I), e(R, I), e(R, 2 * I)
        self.scaled_d, self.scaled_f = e(R, d), e(R, 2 * I)
        self.rlogits, self.drl = e(tokens, E), e(tokens, E)
        self.idx = torch.zeros(tokens, top_k, **i32)
        self.wts = torch.zeros(tokens, top_k, **f32)
        self.probs = torch.zeros(tokens, E, **f32)
        self.dwts = torch.zeros(tokens, top_k, **f32)
        self.entry_rank, self.entry_pos = torch.zeros(n, **i32), torch.zeros(n, **i32)
        self.tile_group = torch.full((R // 128,), -1, **i32)
        self.gk_expert = torch.zeros(El, 2, **i32)
        self.gk_src = torch.zeros(El * ctx.world, 2, **i32)
        self.row_src = torch.full((R,), -1, **i32)
        self.rows_total = torch.zeros(1, **i32)
        self.ss = torch.zeros(2, El * ctx.world, dtype=torch.float64, device=dev)
        self.epoch = 0
        self.x = None
        self._one = self._gwd = self._gwgu = None

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                sync_before: bool = True) -> torch.Tensor:
        """``out = residual + sum_slot w * expert(x)``. ``sync_before`` separates this call from the group's previous
        use of the layer's receive buffers (a peer may still be in the backward of the previous example)."""
        c, L, s = self.ctx, _L(), self.ctx._s()
        T, k, d, n = self.T, self.k, self.d, self.ctx.n_entries
        if x.shape != (T, d) or x.dtype != _bf16:
            raise ValueError(f"expected a [{T}, {d}] bf16 activation")
        if sync_before:
            c.barrier()
        c.epoch += 1
        ep = self.epoch = c.epoch
        err = _p(c.err)
        G.gemm(x, self.router_w, out=self.rlogits)
        _lib.check(L.opk_moe_route(_p(self.rlogits), self.rlogits.stride(0), T, self.E, k, int(self.norm_topk), _p(self.idx),
                                   _p(self.wts), _p(self.probs), s), "moe_route")
        _lib.check(L.opk_ep_count(c.g, _p(self.idx), n, _p(self.entry_rank), ep, s), "ep_count")
        _lib.check(L.opk_ep_dispatch(c.g, self.recv_x_peers, _p(x), x.stride(0), k, None, _p(self.idx), _p(self.entry_rank),
                                     _p(self.entry_pos), 0, n, d, PHASE_COUNTS, PHASE_ROWS, ep, err, s), "ep_dispatch")
        _lib.check(L.opk_ep_prepare(c.g, PHASE_ROWS, ep, _p(self.tile_group), _p(self.gk_expert), _p(self.gk_src),
                                    _p(self.row_src), _p(self.rows_total), err, s), "ep_prepare")
        _lib.check(L.opk_ep_zero_pad(_p(self.recv_x), _p(self.row_src), _p(self.rows_total), c.r_cap, d, s), "ep_zero_pad")
        G.gemm(self.recv_x, self.wgu, out=self.gu, epilogue=G.EPI_SWIGLU, act=self.act, tile_group=self.tile_group)
        G.gemm(self.act, self.wd, out=self.ye, tile_group=self.tile_group)
        _lib.check(L.opk_ep_signal(c.g, PHASE_OUT, ep, s), "ep_signal")
        if out is None:
            out = torch.empty(T, d, dtype=_bf16, device=x.device)
        _lib.check(L.opk_ep_combine(c.g, self.ye_peers, _p(self.entry_pos), _p(self.wts), k, _p(residual), T, d, _p(out),
                                    PHASE_OUT, ep, err, s), "ep_combine")
        self.x = x
        return out

    # ------------------------------------------------------------------ backward, pass 1
    def backward(self, dy: torch.Tensor, *, router_grad_out: torch.Tensor | None = None, sumsq: torch.Tensor | None = None,
                 dx_out: torch.Tensor | None = None):
        """Returns ``(dx, d_router, expert_sq_norms)``: input gradient and router weight gradient of THIS rank's
        example, and for every source rank the squared norm of its example's gradient w.r.t. the local experts
        (float64 ``[world]``). No expert weight gradient is stored; see :meth:`accumulate_clipped`."""
        c, L, s = self.ctx, _L(), self.ctx._s()
        T, k, d, n = self.T, self.k, self.d, self.ctx.n_entries
        # the backward phases take a fresh epoch: layers run backward in the opposite order of their forward epochs,
        # and a flag wait is "flag >= epoch", so reusing the forward epoch would let a layer pass on a later layer's flag
        c.epoch += 1
        ep = c.epoch
        err = _p(c.err)
        x = self.x
        # d(combination weights) needs the expert outputs of the owners; the upstream rows go out weighted
        _lib.check(L.opk_ep_combine_bwd(self.ye_peers, _p(dy), _p(self.entry_pos), n, k, d, _p(self.dwts), s), "ep_combine_bwd")
        _lib.check(L.opk_ep_dispatch(c.g, self.dy_peers, _p(dy), dy.stride(0), k, _p(self.wts), None, None, _p(self.entry_pos),
                                     1, n, d, -1, PHASE_DROWS, ep, err, s), "ep_dispatch")
        _lib.check(L.opk_ep_wait(c.g, PHASE_DROWS, ep, err, s), "ep_wait")
        _lib.check(L.opk_ep_zero_pad(_p(self.dy_rows), _p(self.row_src), _p(self.rows_total), c.r_cap, d, s), "ep_zero_pad")
        self.ss.zero_()
        # squared norms per (local expert, source example): grouped weight-gradient GEMMs that only reduce sum(C^2)
        G.gemm(self.dy_rows, self.act, a_mn=True, b_mn=True, epilogue=G.EPI_SUMSQ, sumsq=self.ss[0], group_k=self.gk_src,
               norm_only=True)
        G.swiglu_dgrad(self.dy_rows, self.wd, self.gu, out=self.dgu, tile_group=self.tile_group)
        G.gemm(self.dgu, self.recv_x, a_mn=True, b_mn=True, epilogue=G.EPI_SUMSQ, sumsq=self.ss[1], group_k=self.gk_src,
               norm_only=True)
        G.gemm(self.dgu, self.wgu, b_mn=True, out=self.dxs, tile_group=self.tile_group)
        _lib.check(L.opk_ep_signal(c.g, PHASE_DOUT, ep, s), "ep_signal")
        norms = self.ss.sum(0).view(self.El, c.world).sum(0)
        dx = dx_out if dx_out is not None else torch.empty(T, d, dtype=_bf16, device=dy.device)
        _lib.check(L.opk_ep_combine(c.g, self.dxs_peers, _p(self.entry_pos), None, k, None, T, d, _p(dx), PHASE_DOUT, ep, err, s),
                   "ep_combine")
        # router (replicated weight, this rank's example only)
        _lib.check(L.opk_moe_route_bwd(_p(self.probs), _p(self.idx), _p(self.dwts), T, self.E, k, int(self.norm_topk),
                                       _p(self.drl), self.drl.stride(0), s), "moe_route_bwd")
        # ``router_grad_out`` / ``sumsq``: the caller's per-example gradient slot and squared-norm accumulator
        d_router = G.linear_wgrad(self.drl, x, out=router_grad_out, sumsq=sumsq)
        G.gemm(self.drl, self.router_w, b_mn=True, out=dx, residual=dx)
        return dx, d_router, norms

    # ------------------------------------------------------------------ backward, pass 2
    def accumulate_clipped(self, scales: torch.Tensor, acc_wgu: torch.Tensor, acc_wd: torch.Tensor) -> None:
        """``acc += sum_b scales[b] * dW^(b)`` for the local experts (``scales`` float32, indexed by source rank):
        the clip factor of the example a row belongs to is folded into the GEMM operand rows."""
        c, L, s = self.ctx, _L(), self.ctx._s()
        scales = scales.to(torch.float32).contiguous()
        _lib.check(L.opk_ep_scale_rows(_p(self.dy_rows), _p(self.row_src), _p(scales), c.r_cap, self.d, _p(self.scaled_d), s),
                   "ep_scale_rows")
        _lib.check(L.opk_ep_scale_rows(_p(self.dgu), _p(self.row_src), _p(scales), c.r_cap, 2 * self.I, _p(self.scaled_f), s),
                   "ep_scale_rows")
        from ..ops import kernels as K

        if self._one is None:
            self._one = torch.ones(1, dtype=torch.float32, device=self.gu.device)
            self._gwd = torch.empty(self.El, self.d, self.I, dtype=_bf16, device=self.gu.device)
            self._gwgu = torch.empty(self.El, 2 * self.I, self.d, dtype=_bf16, device=self.gu.device)
        G.gemm(self.scaled_d, self.act, a_mn=True, b_mn=True, group_k=self.gk_expert, out=self._gwd)
        G.gemm(self.scaled_f, self.recv_x, a_mn=True, b_mn=True, group_k=self.gk_expert, out=self._gwgu)
        K.clip_accumulate(self._gwd.view(-1), self._one, acc_wd.view(-1))
        K.clip_accumulate(self._gwgu.view(-1), self._one, acc_wgu.view(-1))
