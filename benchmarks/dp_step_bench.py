"""Device-timed optimizer step of the sharded engine on N GPUs, against the HBM and NVLink rooflines.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m benchmarks.dp_step_bench [--model llama32_1b] [--iters 5]

For every shard mode the engine's own ``apply_update()`` (barriers, the fused ``opk_dp_step`` kernel, zeroing of the
sums) is timed with CUDA events on the launching stream after warm-up, as the maximum over ranks, on the engine's
real buffers (their total is far larger than L2). Modes:

``state``  sums and parameters replicated, moments sharded: the kernel reduce-scatters by loading every peer's fp32
           sums over NVLink and all-gathers by storing the new bf16 parameters into every replica.
``full``   sums and parameters sharded as well: the reduction happened during the backward (pushes into the owners'
           shards) and non-owners fetch parameters in their next forward, so the step touches local memory only.
``nccl``   the same step on library collectives: NCCL reduce-scatter, local step kernel, NCCL all-gather.

Per mode one JSON line: time, bytes through this GPU's HBM and over its NVLink ports (from the algorithm, per rank),
and achieved / roofline where the roofline is the slower of bytes / measured HBM copy rate and link bytes / 770 GB/s
(the measured peer-copy rate per direction).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def _hbm_gbs() -> tuple[float, str]:
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "MEASURED_PEAKS.json")
    try:
        with open(path, encoding="utf-8") as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama32_1b")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--modes", default="state,full,nccl")
    a = ap.parse_args()
    from opake_b200.parallel import comm

    rank, world, local = comm.init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    from opake_b200.models import config as C
    from opake_b200.ops._lib import raise_if_device_error
    from opake_b200.parallel.engine import EngineConfig, ShardedDPEngine

    mcfg = getattr(C, a.model)()
    hbm, src = _hbm_gbs()
    for mode in a.modes.split(","):
        if mode == "nccl" and world == 1:
            continue
        kw = dict(shard_params=mode == "full", shard_sums=mode == "full", comm_backend="nccl" if mode == "nccl" else "peer")
        eng = ShardedDPEngine(mcfg, EngineConfig(logical_batch=world, noise_multiplier=0.9, use_cuda_graph=False, seq_len=128, **kw), dev)
        P, n = eng.layout.total, eng.shard_len
        eng.acc.normal_()                      # something to reduce; the step's cost does not depend on the values
        for _ in range(3):
            eng.apply_update()
        torch.cuda.synchronize(dev)
        times = []
        for _ in range(a.iters):
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.apply_update()
            e1.record()
            torch.cuda.synchronize(dev)
            times.append(e0.elapsed_time(e1))
        raise_if_device_error(dev)
        t = torch.tensor(sorted(times)[len(times) // 2], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
        # bytes per rank, from the algorithm: moments 16 n (read + write), parameter read 2 n; mode-specific rest
        if mode == "state":
            hbm_b = 16 * n + 2 * n + 4 * n + 2 * n + 4 * P + 4 * n * (world - 1) + 2 * n * (world - 1)
            #        m,v      p read  own sum  own p   zero    peers read my sums   peers write my replica
            link_in, link_out = 4 * n * (world - 1), 2 * n * (world - 1)
        elif mode == "full":
            hbm_b = 16 * n + 2 * n + 4 * n + 4 * n + 2 * n          # m,v; p read; sum read; sum zero; p write
            link_in = link_out = 0
        else:
            hbm_b = 16 * n + 2 * n + 4 * n + 2 * n + 4 * P + 4 * P + 4 * n + 2 * n * world
            link_in, link_out = 4 * n * (world - 1) + 2 * n * (world - 1), 4 * n * (world - 1) + 2 * n * (world - 1)
        t_hbm, t_link = hbm_b / (hbm * 1e9), max(link_in, link_out) / (LINK_GBS * 1e9)
        roof_ms = max(t_hbm, t_link) * 1e3
        if rank == 0:
            print(json.dumps({"case": "dp_step", "mode": mode, "world": world, "model": mcfg.name, "params": P, "shard": n,
                              "ms": round(ms, 3), "hbm_bytes_per_rank": hbm_b, "link_bytes_in": link_in, "link_bytes_out": link_out,
                              "roofline_ms": round(roof_ms, 3), "bound": "link" if t_link > t_hbm else "hbm",
                              "frac_of_roofline": round(roof_ms / ms, 3), "hbm_gbs_used": hbm, "hbm_source": src,
                              "link_gbs_used": LINK_GBS}), flush=True)
        del eng
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
