"""Linear layers whose weight stays sharded over the ranks: the all-gather is fused into the consuming GEMM.

Each rank stores ``N / world`` rows of a ``[N, K]`` weight in peer-addressable memory. ``forward`` computes
``x @ W.T`` as ``world`` tcgen05 GEMMs, one per shard, whose B operand is the peer's shard itself. For products with
at least 256 rows the two-CTA kernel runs with four extra warps per CTA that copy the remote shard over NVLink into a
local scratch matrix, one band of 2048 weight rows at a time, while the tensor-core warps consume the bands that
have arrived (per-band counters, bounded waits): every remote byte crosses NVLink once, no collective is called and
the transfer overlaps the math band by band inside one kernel. Smaller products let the TMA producer pull tiles
straight from the remote memory. Shards are visited starting with
the local one and continuing with rank+1, rank+2, ... so that at any moment the ranks read from different peers.
The loads are ordinary TMA tile loads that each CTA issues for itself.

The weight gradient of a row-sharded weight is local (``dW_s = dy[:, rows_s].T @ x`` is needed only by the owner
when the ranks work on the same ``x``; under data parallelism it is followed by the reduce-scatter of the optimizer
step), and the input gradient sums the shards' contributions, again by reading peer shards in place.

This serves models whose bf16 parameters do not fit replicated. The benchmarked engine keeps a bf16 replica per GPU
(16 GB for an 8B model on a 180 GB part) because its per-example schedule re-reads the weights for every example,
which NVLink (0.77 TB/s measured) cannot feed as HBM (6.5 TB/s) does.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import gemm as G
from . import comm

__all__ = ["ShardedWeight", "sharded_linear_forward", "sharded_linear_dgrad"]


class ShardedWeight:
    def __init__(self, n_out: int, n_in: int, device: torch.device, group=None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_out % (8 * self.world) or n_in % 8:
            raise ValueError("rows per shard and the reduction size must be multiples of 8")
        self.n_out, self.n_in, self.rows = n_out, n_in, n_out // self.world
        self.buf = comm.alloc_peer_buffer(self.rows * n_in, torch.bfloat16, device, group)
        self.local = self.buf.local.view(self.rows, n_in)
        self.shards = [self.local if r == self.rank else self.buf.peer_view(r, (self.rows, n_in)) for r in range(self.world)]
        self._scratch = None

    def scratch(self):
        """Local staging matrix for ONE remote shard plus its band counters (created on first use, reused for every
        remote shard in turn: the products are ordered on one stream)."""
        if self._scratch is None:
            dev = self.local.device
            self._scratch = (torch.empty(self.rows, self.n_in, dtype=torch.bfloat16, device=dev),
                             torch.zeros((max(self.rows, self.n_in) + 2047) // 2048, dtype=torch.int32, device=dev))
        return self._scratch

    def order(self) -> list[int]:
        return [(self.rank + i) % self.world for i in range(self.world)]

    def publish(self) -> None:
        """Makes local writes to the shard visible to the peers' next kernels (stream-ordered device barrier)."""
        self.buf.barrier()


def sharded_linear_forward(x: torch.Tensor, w: ShardedWeight, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x [M, K]`` -> ``[M, N]``; every column block is produced from the shard that owns it, read in place."""
    M = x.shape[0]
    if out is None:
        out = torch.empty(M, w.n_out, dtype=torch.bfloat16, device=x.device)
    staged = M >= 256 and w.rows > 128 and G.pair_mode()
    for s in w.order():
        remote = s != w.rank
        # a remote shard is copied once, band by band, by extra warps of the GEMM kernel itself while its tensor-core
        # warps work on the bands that have arrived; reading it directly would fetch every tile once per row tile
        G.gemm(x, w.shards[s], out=out[:, s * w.rows:(s + 1) * w.rows], stage=w.scratch() if (remote and staged) else None)
    return out


def sharded_linear_dgrad(dy: torch.Tensor, w: ShardedWeight, out: torch.Tensor | None = None) -> torch.Tensor:
    """``dx = dy @ W`` summed over shards (``dy [M, N]``)."""
    M = dy.shape[0]
    if out is None:
        out = torch.empty(M, w.n_in, dtype=torch.bfloat16, device=dy.device)
    first = True
    staged = M >= 256 and w.n_in > 128 and G.pair_mode()
    for s in w.order():
        G.gemm(dy[:, s * w.rows:(s + 1) * w.rows], w.shards[s], b_mn=True, out=out, residual=None if first else out,
               stage=w.scratch() if (s != w.rank and staged) else None)
        first = False
    return out
