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
    a = ap.parse_args()
    rank, world, local = comm.init_distributed()
    dev = torch.device("cuda", local)
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


if __name__ == "__main__":
    main()
