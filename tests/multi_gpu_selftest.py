"""Multi-rank self-test of the sharded engine: ``torchrun ... -m tests.multi_gpu_selftest --out file.pt``.

Runs two DP steps of a tiny decoder on a fixed logical batch split over the ranks and stores the resulting parameters
(rank 0). Comparing the files of a 1-rank and an N-rank run checks the fused reduce-scatter / noise / AdamW / all-gather
kernel: with the same keys both runs must produce the same parameters up to summation order.
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from opake_b200.models.config import tiny_llama
from opake_b200.parallel import comm
from opake_b200.parallel.engine import EngineConfig, ShardedDPEngine


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--blt", action="store_true")
    ap.add_argument("--toeplitz", action="store_true", help="banded Toeplitz correlated noise (band-MF / banded square root)")
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--shard-params", action="store_true", help="owners keep the parameters; fetched inside the forward GEMMs")
    ap.add_argument("--shard-sums", action="store_true", help="fp32 sums sharded, accumulation groups reduce-scattered")
    ap.add_argument("--graph", action="store_true", help="run the examples through CUDA graphs")
    ap.add_argument("--comm", default="peer", choices=["peer", "nccl"], help="optimizer-step communication backend")
    ap.add_argument("--ep-train", action="store_true",
                    help="train a tiny mixture-of-experts decoder: all experts local on one rank, expert parallel on several")
    ap.add_argument("--sharded-linear", action="store_true", help="check the sharded-weight GEMMs instead of the engine")
    ap.add_argument("--ep-fused", action="store_true", help="check the expert-parallel dispatch / combine kernels")
    ap.add_argument("--sharded-linear-bench", action="store_true",
                    help="time the sharded-weight GEMM (peer shards read in place) against the same GEMM on a local weight")
    a = ap.parse_args()
    rank, world, local = comm.init_distributed()
    dev = torch.device("cuda", local)
    if a.sharded_linear:
        _sharded_linear_check(rank, world, dev, a.out)
        return
    if a.sharded_linear_bench:
        _sharded_linear_bench(rank, world, dev, a.out)
        return
    if a.ep_fused:
        res = ep_fused_check(rank, world, dev)
        if rank == 0:
            torch.save(res, a.out)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if a.ep_train:
        _ep_train(rank, world, dev, a)
        return
    cfg = tiny_llama()
    if a.seq > cfg.max_seq:
        cfg = tiny_llama(max_seq=a.seq)
    ecfg = EngineConfig(logical_batch=a.batch, noise_multiplier=0.7, lr=1e-2, seed=5, use_cuda_graph=a.graph,
                        blt_decay=(0.9, 0.5) if a.blt else (), blt_scale=(0.3, 0.2) if a.blt else (),
                        toeplitz_coef=(1.0, 0.5, 0.375, 0.3125) if a.toeplitz else (),
                        shard_params=a.shard_params, shard_sums=a.shard_sums, accumulate_group=2, comm_backend=a.comm)
    eng = ShardedDPEngine(cfg, ecfg, dev)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (a.batch, a.seq), generator=g, dtype=torch.int32)
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
    eng.gather_params()
    torch.cuda.synchronize()
    from opake_b200.ops._lib import raise_if_device_error

    raise_if_device_error(dev)
    if rank == 0:
        staged = sorted(eng._refresh_plan(a.seq)[0]) if eng.shard_params else []
        torch.save({"params": eng.params.float().cpu(), "losses": losses, "world": world, "staged": staged,
                    "bounds": list(eng.bounds)}, a.out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _ep_train(rank: int, world: int, dev: torch.device, a) -> None:
    """DP steps of a tiny mixture-of-experts decoder without noise. On one rank every expert is local (grouped GEMMs
    inside the flat runtime); on several ranks the experts are sharded and tokens travel (expert-parallel layers,
    two-pass clipping across ranks). Same logical batch, same initial weights: the losses of every step and the final
    router and expert weights must agree."""
    from opake_b200.ops._lib import raise_if_device_error

    cfg = tiny_llama(n_experts=8, top_k=2, expert_ffn=64, d_model=128, n_heads=2, n_kv_heads=2, head_dim=64, ffn=0, max_seq=256,
                     name="tiny-moe", family="olmoe")
    T = 256
    # plain SGD: the update is linear in the summed gradient, so differences in summation order stay small (Adam's
    # normalised update flips sign on near-zero gradient entries)
    ecfg = EngineConfig(logical_batch=a.batch, noise_multiplier=0.0, clip_norm=0.5, lr=20.0, optimizer="sgd", weight_decay=0.0,
                        seed=5, use_cuda_graph=a.graph, accumulate_group=2, expert_parallel=True, seq_len=T)
    eng = ShardedDPEngine(cfg, ecfg, dev)
    def snapshot():
        views = eng.layout.views(eng.params)
        routers = torch.stack([views[f"layers.{i}.router"].float().cpu() for i in range(cfg.n_layers)])
        if eng.ep is None:
            wgu = torch.stack([views[f"layers.{i}.experts.wgu"].float().cpu() for i in range(cfg.n_layers)])
            wd = torch.stack([views[f"layers.{i}.experts.wd"].float().cpu() for i in range(cfg.n_layers)])
        else:
            parts = [torch.empty_like(eng.ep.params) for _ in range(world)]
            dist.all_gather(parts, eng.ep.params)
            wgu_l, wd_l = [], []
            for i in range(cfg.n_layers):
                per_rank = [eng.ep.views(p, i) for p in parts]
                wgu_l.append(torch.cat([v[0] for v in per_rank]).float().cpu())
                wd_l.append(torch.cat([v[1] for v in per_rank]).float().cpu())
            wgu, wd = torch.stack(wgu_l), torch.stack(wd_l)
        wqkv = views["layers.0.wqkv"].float().cpu()
        return {"routers": routers, "wgu": wgu, "wd": wd, "wqkv": wqkv}

    before = snapshot()
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (a.batch, T), generator=g, dtype=torch.int32)
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
    raise_if_device_error(dev)
    after = snapshot()
    c = eng.runtime.clip_count.clone().to(torch.int64)
    if world > 1:
        dist.all_reduce(c)
    if rank == 0:
        torch.save({"losses": losses, "world": world, "clipped": int(c.item()), "init": before,
                    "delta": {k: after[k] - before[k] for k in after}}, a.out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _sharded_linear_check(rank: int, world: int, dev: torch.device, out: str) -> None:
    """Every rank builds the same full weight, keeps its row shard in peer memory, and compares the sharded forward
    and input-gradient GEMMs (peer shards read in place) with the full-weight products."""
    from opake_b200.parallel.sharded_linear import ShardedWeight, sharded_linear_dgrad, sharded_linear_forward
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



def _sharded_linear_bench(rank: int, world: int, dev: torch.device, out: str, M: int = 2048, N: int = 28672, Kd: int = 4096,
                          iters: int = 10) -> None:
    """Llama-3-8B gate/up projection with the weight row-sharded over the ranks: device time of the sharded forward
    (``world`` GEMMs, ``world - 1`` of them fed by TMA loads from a peer's memory over NVLink) against the same product
    on a local full weight. Maximum over ranks; a 256 MB buffer is overwritten before every timed call. The NVLink
    roofline is the bytes of the remote shards divided by 770 GB/s (measured peer-copy bandwidth per direction)."""
    import json

    from opake_b200.parallel.sharded_linear import ShardedWeight, sharded_linear_forward
    from opake_b200.ops import gemm as G

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(M, Kd, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    sw = ShardedWeight(N, Kd, dev)
    sw.local.normal_(0, 0.05)
    sw.publish()
    full = torch.randn(N, Kd, device=dev).mul_(0.05).to(torch.bfloat16)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            if world > 1:
                sw.publish()                     # ranks start each call together
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_.record()
            fn()
            b_.record()
            torch.cuda.synchronize(dev)
            ts.append(a_.elapsed_time(b_) * 1e3)
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    from opake_b200.parallel.sharded_linear import sharded_linear_dgrad

    t_sharded = timed(lambda: sharded_linear_forward(x, sw, out=y))
    t_local = timed(lambda: G.gemm(x, full, out=y))
    dy = torch.randn(M, N, device=dev).mul_(0.1).to(torch.bfloat16)
    dx = torch.empty(M, Kd, dtype=torch.bfloat16, device=dev)
    t_dgrad = timed(lambda: sharded_linear_dgrad(dy, sw, out=dx))
    t_dgrad_local = timed(lambda: G.gemm(dy, full, b_mn=True, out=dx))
    remote_bytes = (world - 1) / world * N * Kd * 2
    res = {"case": "sharded_linear_forward", "world": world, "M": M, "N": N, "K": Kd, "sharded_us": round(t_sharded, 1),
           "local_weight_us": round(t_local, 1), "tflops_sharded": round(2.0 * M * N * Kd / t_sharded / 1e6, 1),
           "nvlink_roofline_us": round(remote_bytes / 770e3, 1),
           "roofline_us": round(max(remote_bytes / 770e3, t_local), 1),
           "dgrad_sharded_us": round(t_dgrad, 1), "dgrad_local_weight_us": round(t_dgrad_local, 1)}
    if world > 1:
        sw.publish()
    if rank == 0:
        print(json.dumps(res))
        torch.save(res, out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def ep_fused_check(rank: int, world: int, dev: torch.device, T: int = 256, d: int = 128, I: int = 64, E: int = 8, k: int = 2,
                   calls: int = 2) -> dict:
    """Runs the fused expert-parallel layer (forward, backward with per-source norms, clipped accumulation) and
    compares every result with a dense fp32 autograd computation that uses the layer's own routing decisions.
    Every rank generates all ranks' inputs, so the oracle needs no communication beyond gathering the routing."""
    import torch.nn.functional as F

    from opake_b200.ops._lib import raise_if_device_error
    from opake_b200.parallel.ep_fused import EpContext, FusedExpertParallelLayer

    gen = torch.Generator().manual_seed(11)
    bf = lambda t: t.to(torch.bfloat16).to(dev)
    router = bf(torch.randn(E, d, generator=gen) * 0.5)
    wgu = bf(torch.randn(E, 2 * I, d, generator=gen) * 0.1)      # gate / up rows interleaved
    wd = bf(torch.randn(E, d, I, generator=gen) * 0.1)
    El = E // world
    mine = slice(rank * El, (rank + 1) * El)
    ctx = EpContext(E, T * k, dev)
    layer = FusedExpertParallelLayer(ctx, router, wgu[mine].contiguous(), wd[mine].contiguous(), T, k)
    worst = {"out": 0.0, "dx": 0.0, "d_router": 0.0, "norms": 0.0, "acc_wgu": 0.0, "acc_wd": 0.0}

    def rel(a, b):
        return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12)).item()

    for _ in range(calls):                                       # the second call reuses every buffer and flag
        xs = bf(torch.randn(world, T, d, generator=gen))
        dys = bf(torch.randn(world, T, d, generator=gen))
        scales = torch.tensor([0.5, 0.25, 1.0, 0.125, 0.75, 0.3, 0.9, 0.6][:world], device=dev)
        x, dy = xs[rank].contiguous(), dys[rank].contiguous()
        out = layer.forward(x, residual=x)
        dx, d_router, norms = layer.backward(dy)
        acc_wgu = torch.zeros(El, 2 * I, d, dtype=torch.float32, device=dev)
        acc_wd = torch.zeros(El, d, I, dtype=torch.float32, device=dev)
        layer.accumulate_clipped(scales, acc_wgu, acc_wd)
        raise_if_device_error(dev)
        idx_all = [torch.empty_like(layer.idx) for _ in range(world)]
        if world > 1:
            dist.all_gather(idx_all, layer.idx)
        else:
            idx_all = [layer.idx]
        ref_norms = torch.zeros(world, dtype=torch.float64, device=dev)
        ref_wgu, ref_wd = torch.zeros_like(acc_wgu), torch.zeros_like(acc_wd)
        for s in range(world):
            xf = xs[s].float().requires_grad_(True)
            rw, wguf, wdf = (t.float().requires_grad_(True) for t in (router, wgu, wd))
            idx = idx_all[s].long()
            w = (xf @ rw.t()).softmax(-1).gather(1, idx)
            y = xf.clone()
            for slot in range(k):
                for e in range(E):
                    rows = (idx[:, slot] == e).nonzero().squeeze(1)
                    if rows.numel():
                        gu = xf[rows] @ wguf[e].t()
                        h = F.silu(gu[:, 0::2]) * gu[:, 1::2]
                        y = y.index_add(0, rows, (h @ wdf[e].t()) * w[rows, slot].unsqueeze(1))
            gx, gr, gwgu, gwd = torch.autograd.grad((y * dys[s].float()).sum(), (xf, rw, wguf, wdf))
            ref_norms[s] = gwgu[mine].double().pow(2).sum() + gwd[mine].double().pow(2).sum()
            ref_wgu += scales[s] * gwgu[mine]
            ref_wd += scales[s] * gwd[mine]
            if s == rank:
                worst["out"] = max(worst["out"], rel(out, y.detach()))
                worst["dx"] = max(worst["dx"], rel(dx.float() + dy.float(), gx))   # oracle includes the residual path
                worst["d_router"] = max(worst["d_router"], rel(d_router, gr))
        worst["norms"] = max(worst["norms"], ((norms - ref_norms).abs() / (ref_norms + 1e-12)).max().item())
        worst["acc_wgu"] = max(worst["acc_wgu"], rel(acc_wgu, ref_wgu))
        worst["acc_wd"] = max(worst["acc_wd"], rel(acc_wd, ref_wd))
    errs = torch.tensor(list(worst.values()), device=dev)
    if world > 1:
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    return {"world": world, **{name: v for name, v in zip(worst, errs.tolist())}}

if __name__ == "__main__":
    main()
