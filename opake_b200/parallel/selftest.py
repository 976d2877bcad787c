"""Multi-rank self-test of the sharded engine: ``torchrun ... -m opake_b200.parallel.selftest --out file.pt``.

Runs two DP steps of a tiny decoder on a fixed logical batch split over the ranks and stores the resulting parameters
(rank 0). Comparing the files of a 1-rank and an N-rank run checks the fused reduce-scatter / noise / AdamW / all-gather
kernel: with the same keys both runs must produce the same parameters up to summation order.
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from ..models.config import tiny_llama
from . import comm
from .engine import EngineConfig, ShardedDPEngine


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--blt", action="store_true")
    ap.add_argument("--sharded-linear", action="store_true", help="check the sharded-weight GEMMs instead of the engine")
    a = ap.parse_args()
    rank, world, local = comm.init_distributed()
    dev = torch.device("cuda", local)
    if a.sharded_linear:
        _sharded_linear_check(rank, world, dev, a.out)
        return
    cfg = tiny_llama()
    ecfg = EngineConfig(logical_batch=a.batch, noise_multiplier=0.7, lr=1e-2, seed=5, use_cuda_graph=False,
                        blt_decay=(0.9, 0.5) if a.blt else (), blt_scale=(0.3, 0.2) if a.blt else ())
    eng = ShardedDPEngine(cfg, ecfg, dev)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (a.batch, 128), generator=g, dtype=torch.int32)
    labels = torch.roll(tok, -1, 1).clone()
    labels[:, -1] = -100
    per = a.batch // world
    mine = slice(rank * per, (rank + 1) * per)
    losses = []
    for _ in range(a.steps):
        l = eng.step(tok[mine].pin_memory(), labels[mine].pin_memory())
        if world > 1:
            dist.all_reduce(l)
        losses.append(l.item() / a.batch)
    torch.cuda.synchronize()
    if rank == 0:
        torch.save({"params": eng.params.float().cpu(), "losses": losses, "world": world}, a.out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _sharded_linear_check(rank: int, world: int, dev: torch.device, out: str) -> None:
    """Every rank builds the same full weight, keeps its row shard in peer memory, and compares the sharded forward
    and input-gradient GEMMs (peer shards read in place) with the full-weight products."""
    from .sharded_linear import ShardedWeight, sharded_linear_dgrad, sharded_linear_forward
    N, Kd, M = 1024, 512, 384
    g = torch.Generator().manual_seed(3)
    W = (torch.randn(N, Kd, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    x = (torch.randn(M, Kd, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    dy = (torch.randn(M, N, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    sw = ShardedWeight(N, Kd, dev)
    sw.local.copy_(W[rank * sw.rows:(rank + 1) * sw.rows])
    sw.publish()
    y = sharded_linear_forward(x, sw)
    dx = sharded_linear_dgrad(dy, sw)
    torch.cuda.synchronize()
    e1 = ((y.float() - x.float() @ W.float().t()).abs().max() / (x.float() @ W.float().t()).abs().max()).item()
    e2 = ((dx.float() - dy.float() @ W.float()).abs().max() / (dy.float() @ W.float()).abs().max()).item()
    errs = torch.tensor([e1, e2], device=dev)
    if world > 1:
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        sw.publish()          # nobody frees its shard while a peer may still read it
    if rank == 0:
        torch.save({"fwd_err": errs[0].item(), "dgrad_err": errs[1].item(), "world": world}, out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
