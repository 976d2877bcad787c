"""Times the expert-parallel exchange: fused peer-memory kernels against ``all_to_all_single``.

``torchrun --nproc-per-node N -m benchmarks.ep_bench`` (OLMoE-1B-7B layer shape by default: 2048 tokens per
rank, d = 2048, 64 experts, top-8). Both arms move the same rows: dispatch = every (token, slot) entry's activation row
to the rank that owns its expert, grouped by expert there; combine = the expert output rows back, summed over the slots
with the routing weights. The library arm is what a framework without its own kernels does: exchange the split sizes,
read them on the host, sort, gather, ``all_to_all_single``, and the mirror image on the way back. Device time per
call (CUDA events), maximum over ranks. Rank 0 prints one JSON line with both times and the NVLink roofline of the
fused arm (bytes that must leave a rank / measured peer-copy bandwidth of 770 GB/s per direction).
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from opake_b200.ops import _lib
from opake_b200.parallel import comm
from opake_b200.parallel.ep_fused import PHASE_COUNTS, PHASE_OUT, PHASE_ROWS, EpContext, _L, _p

PEER_COPY_GBS = 770.0


def _time(fn, iters: int, warmup: int, dev) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    if dist.is_initialized():
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e3   # microseconds


def _layer_bench(a, rank: int, world: int, dev) -> None:
    """One OLMoE-shaped MoE layer with the experts sharded over the ranks, one example (``tokens`` rows) per rank:
    device time of forward, of backward pass 1 (input gradients + per-source squared norms) and of pass 2 (clipped
    accumulation of the expert weight gradients), maximum over ranks. FLOPs counted: 3 products per pass direction
    over the routed rows (gate/up, down; forward, input gradient, weight gradient twice: norms and accumulation)."""
    from opake_b200.parallel.ep_fused import FusedExpertParallelLayer

    T, d, E, k, I = a.tokens, a.d, a.experts, a.top_k, a.ffn
    El = E // world
    gen = torch.Generator().manual_seed(5 + rank)
    bf = lambda t: t.to(torch.bfloat16).to(dev)
    router = bf(torch.randn(E, d, generator=torch.Generator().manual_seed(1)) * 0.05)
    wgu = bf(torch.randn(El, 2 * I, d, generator=gen) * 0.02)
    wd = bf(torch.randn(El, d, I, generator=gen) * 0.02)
    ctx = EpContext(E, T * k, dev)
    layer = FusedExpertParallelLayer(ctx, router, wgu, wd, T, k)
    x, dy = bf(torch.randn(T, d, generator=gen)), bf(torch.randn(T, d, generator=gen) * 0.1)
    scales = torch.full((world,), 0.5, device=dev)
    acc_wgu = torch.zeros(El, 2 * I, d, dtype=torch.float32, device=dev)
    acc_wd = torch.zeros(El, d, I, dtype=torch.float32, device=dev)
    out = torch.empty(T, d, dtype=torch.bfloat16, device=dev)
    t_fwd = _time(lambda: layer.forward(x, residual=x, out=out), a.iters, a.warmup, dev)

    def fwd_bwd():
        layer.forward(x, residual=x, out=out)
        layer.backward(dy)

    def full():
        fwd_bwd()
        layer.accumulate_clipped(scales, acc_wgu, acc_wd)

    t_fb = _time(fwd_bwd, a.iters, a.warmup, dev)
    t_all = _time(full, a.iters, a.warmup, dev)
    _lib.raise_if_device_error(dev)
    rows = T * k                                        # routed rows per rank on average
    flops = 2.0 * rows * d * 3 * I * 5                  # fwd, dgrad, wgrad (norm pass), wgrad (accumulate) + swiglu pairs
    if rank == 0:
        print(json.dumps({"case": "ep_layer", "world": world, "tokens_per_rank": T, "d": d, "experts": E, "top_k": k, "ffn": I,
                          "forward_us": round(t_fwd, 1), "forward_backward_us": round(t_fb, 1),
                          "with_clipped_accumulation_us": round(t_all, 1),
                          "expert_tflops_per_gpu": round(flops / t_all / 1e6, 1),
                          "tokens_per_s_per_layer_all_ranks": round(world * T / (t_all * 1e-6))}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--d", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--phases", action="store_true", help="also report the device time of every kernel of the fused arm")
    ap.add_argument("--layer", action="store_true",
                    help="time a whole expert-parallel MoE layer instead (forward, backward with per-source norms, clipped "
                         "accumulation) on the native kernels")
    ap.add_argument("--ffn", type=int, default=1024, help="expert hidden size for --layer")
    a = ap.parse_args()
    rank, world, local = comm.init_distributed()
    dev = torch.device("cuda", local)
    if a.layer:
        _layer_bench(a, rank, world, dev)
        return
    T, d, E, k = a.tokens, a.d, a.experts, a.top_k
    n = T * k
    gen = torch.Generator().manual_seed(3 + rank)
    x = torch.randn(T, d, generator=gen).to(torch.bfloat16).to(dev)
    idx = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(T)]).to(torch.int32).to(dev)
    wts = torch.rand(T, k, generator=gen).to(dev)

    # ---------------------------------------------------------------- fused arm
    ctx = EpContext(E, n, dev)
    L, s, err = _L(), ctx._s(), _p(ctx.err)
    recv, recv_peers = ctx.rows(d)
    entry_rank = torch.zeros(n, dtype=torch.int32, device=dev)
    entry_pos = torch.zeros(n, dtype=torch.int32, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    tile_group = torch.zeros(ctx.r_cap // 128, **i32)
    gk_e, gk_s = torch.zeros(ctx.e_local, 2, **i32), torch.zeros(ctx.e_local * world, 2, **i32)
    row_src, rows_total = torch.zeros(ctx.r_cap, **i32), torch.zeros(1, **i32)
    out = torch.empty(T, d, dtype=torch.bfloat16, device=dev)

    marks: list = []

    def mark(name):
        if a.phases:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append((name, e))

    def fused():
        mark("start")
        ctx.barrier()
        mark("barrier")
        ctx.epoch += 1
        ep = ctx.epoch
        _lib.check(L.opk_ep_count(ctx.g, _p(idx), n, _p(entry_rank), ep, s), "ep_count")
        mark("count")
        _lib.check(L.opk_ep_dispatch(ctx.g, recv_peers, _p(x), x.stride(0), k, None, _p(idx), _p(entry_rank), _p(entry_pos), 0, n,
                                     d, PHASE_COUNTS, PHASE_ROWS, ep, err, s), "ep_dispatch")
        mark("dispatch")
        _lib.check(L.opk_ep_prepare(ctx.g, PHASE_ROWS, ep, _p(tile_group), _p(gk_e), _p(gk_s), _p(row_src), _p(rows_total), err, s),
                   "ep_prepare")
        mark("prepare")
        _lib.check(L.opk_ep_zero_pad(_p(recv), _p(row_src), _p(rows_total), ctx.r_cap, d, s), "ep_zero_pad")
        # (expert GEMMs would run here on `recv`; the exchange is timed with the received rows as the outputs)
        mark("zero_pad")
        _lib.check(L.opk_ep_signal(ctx.g, PHASE_OUT, ep, s), "ep_signal")
        _lib.check(L.opk_ep_combine(ctx.g, recv_peers, _p(entry_pos), _p(wts), k, None, T, d, _p(out), PHASE_OUT, ep, err, s),
                   "ep_combine")
        mark("signal+combine")

    t_fused = _time(fused, a.iters, a.warmup, dev)
    _lib.raise_if_device_error(dev)
    phases = {}
    if a.phases:      # per-kernel device time of the timed iterations (this rank), microseconds
        per = len(marks) // (a.iters + a.warmup)
        for it in range(a.warmup, a.warmup + a.iters):
            row = marks[it * per:(it + 1) * per]
            for (_, e0), (name, e1) in zip(row[:-1], row[1:]):
                phases[name] = phases.get(name, 0.0) + e0.elapsed_time(e1) * 1e3 / a.iters
        phases = {k_: round(v, 1) for k_, v in phases.items()}
    ref_fused = out.float().clone()

    # ---------------------------------------------------------------- library arm
    El = E // world
    out2 = torch.empty(T, d, dtype=torch.bfloat16, device=dev)

    def library():
        flat = idx.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                    # by expert, therefore by owner rank
        send_counts = torch.bincount(flat // El, minlength=world)
        if world > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts)
            sc, rc = send_counts.tolist(), recv_counts.tolist()     # host synchronisation
        else:
            sc = rc = send_counts.tolist()
        send_x = x[order // k]
        send_e = flat[order]
        if world > 1:
            rx = x.new_empty(sum(rc), d)
            re = flat.new_empty(sum(rc))
            dist.all_to_all_single(rx, send_x, output_split_sizes=rc, input_split_sizes=sc)
            dist.all_to_all_single(re, send_e, output_split_sizes=rc, input_split_sizes=sc)
        else:
            rx, re = send_x, send_e
        by_expert = torch.argsort(re, stable=True)                   # group the received rows by expert
        grouped = rx[by_expert]
        # (expert GEMMs would run here on `grouped`)
        back_rows = torch.empty_like(grouped)
        back_rows[by_expert] = grouped
        if world > 1:
            back = x.new_empty(n, d)
            dist.all_to_all_single(back, back_rows, output_split_sizes=sc, input_split_sizes=rc)
        else:
            back = back_rows
        y = torch.empty_like(back)
        y[order] = back
        out2.copy_((y.view(T, k, d).float() * wts.unsqueeze(-1)).sum(1))

    t_lib = _time(library, a.iters, a.warmup, dev)
    mismatch = (out2.float() - ref_fused).abs().max().item() / (ref_fused.abs().max().item() + 1e-9)
    bytes_out = n * (world - 1) / world * d * 2                       # per direction, per rank, per exchange
    roof = 2 * bytes_out / (PEER_COPY_GBS * 1e3) if world > 1 else 0.0    # microseconds for dispatch + combine
    if rank == 0:
        print(json.dumps({"case": "ep_exchange", "world": world, "tokens": T, "d": d, "experts": E, "top_k": k,
                          "fused_us": round(t_fused, 1), "all_to_all_us": round(t_lib, 1),
                          "speedup": round(t_lib / t_fused, 2), "nvlink_roofline_us": round(roof, 1),
                          "fused_frac_of_roofline": round(roof / t_fused, 3) if world > 1 else None,
                          "arms_mismatch": mismatch, **({"phases_us": phases} if a.phases else {})}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
