"""Headline benchmark: DP tokens/sec for Llama-3-8B-shaped DP-SGD with a sharded optimizer (FSDP-style) on N B200s.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 2 --warmup 3

One step = one DP optimizer step on the logical batch (256 sequences of 2048 tokens, split evenly over the ranks,
processed one example at a time = gradient accumulation), including per-example clipping, the fused
reduce-scatter + Philox noise + AdamW-BC + parameter all-gather kernel. Synthetic Zipf(1.1) tokens, random-init
weights, SFT mask on the first 25 % of each sequence. Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _zipf_tokens(n_seq: int, seq: int, vocab: int, seed: int):
    import numpy as np
    import torch

    rng = np.random.default_rng(seed)
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    p = ranks ** -1.1
    p /= p.sum()
    cdf = np.cumsum(p)
    u = rng.random((n_seq, seq))
    tok = np.searchsorted(cdf, u).clip(0, vocab - 1).astype(np.int32)
    return torch.from_numpy(tok)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_reference(args) -> None:
    """The unmodified reference on the same configuration (``baseline/reference_arm.py``); none of this package is
    imported on that path. Prints the reference's JSON line, or its ``unavailable`` line."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import reference_arm

    reference_arm.run(args)


def run_config_a(args) -> None:
    """CPU plumbing configuration: fp32 DP-SGD on an MLP 784-512-10, 60000 synthetic samples, Poisson q = 256/60000,
    C = 1.0, sigma = 1.1, SGD lr 0.1, 200 steps, PLD accountant at delta = 1e-5 (functional API, no GPU)."""
    import torch
    from torch import nn

    from opake_b200 import accounting as acc
    from opake_b200.dpsgd import PoissonSampler, clipped_grad, gaussian_noise
    from opake_b200.dpsgd import accounting as sgd_acc
    from opake_b200.engine.functional import make_functional
    from opake_b200.engine.random import fold_in, key
    from opake_b200.optimizers import apply_updates, sgd

    steps, n, q, sigma, delta = 200, 60000, 256 / 60000, 1.1, 1e-5
    g = torch.Generator().manual_seed(0)
    x = torch.randn(n, 784, generator=g)
    y = torch.randint(0, 10, (n,), generator=g)
    model = nn.Sequential(nn.Linear(784, 512), nn.ReLU(), nn.Linear(512, 10))
    fmodel, params, _ = make_functional(model, disable_autograd_tracking=True, partition_trainable=True)
    loss_fn = lambda p, xe, ye: nn.functional.cross_entropy(fmodel(p, xe[None]), ye[None])
    grad_fn, cs = clipped_grad(loss_fn, clipping_norm=1.0, normalize_by=256.0, batch_argnums=(1, 2))
    noise_fn, ns = gaussian_noise(noise_multiplier=sigma, key=fold_in(key(0), "noise"))
    opt = sgd(0.1)
    os_ = opt.init(params)
    ledger = acc.Accountant()
    sampler = PoissonSampler(torch.utils.data.TensorDataset(x, y), q, n_steps=steps, key=fold_in(key(0), "sampler"))
    t0, seen = time.perf_counter(), 0
    for idx in sampler:
        clipped, cs = grad_fn(params, x[idx], y[idx], state=cs)
        noised, ns = noise_fn(clipped, ns)
        upd, os_ = opt.update(noised, os_, params=params)
        params = apply_updates(params, upd)
        seen += len(idx)
    dt = time.perf_counter() - t0
    ledger = ledger | sgd_acc.poisson(sgd_acc.gaussian(sigma), q) * steps
    print(json.dumps({"metric": "config a: CPU fp32 DP-SGD MLP 784-512-10, functional API", "value": seen / dt, "unit": "samples/s",
                      "n_gpus": 0, "steps": steps, "higher_is_better": True, "epsilon_at_1e-5": ledger.epsilon_at(delta),
                      "seconds": dt, "dtype": "fp32", "data": "synthetic, seed 0"}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=256, help="logical batch (sequences per optimizer step, all ranks)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--attn", default="auto")
    ap.add_argument("--sigma", type=float, default=0.9)
    ap.add_argument("--blt-buffers", type=int, default=0, help="DP-FTRL: buffered-linear-Toeplitz correlated noise buffers")
    ap.add_argument("--shard", default="auto", choices=["auto", "state", "params", "full"],
                    help="what is sharded over the ranks: 'state' = optimizer moments only (replicated bf16 parameters and fp32 "
                         "sums, all-gather by peer stores in the step kernel); 'params' = also the parameters (fetched inside the "
                         "first forward GEMMs after a step); 'full' = parameters and fp32 sums; 'auto' = full when N > 1")
    ap.add_argument("--comm", default="peer", choices=["peer", "nccl"],
                    help="optimizer-step collectives: 'peer' = this build's kernels over peer memory; 'nccl' = the library baseline "
                         "(reduce-scatter, local step, all-gather), with --shard state")
    ap.add_argument("--group", type=int, default=0, help="gradient buffers per accumulation pass (0 = as many as fit)")
    ap.add_argument("--config", default="d", choices=["a", "b", "c", "d", "e"],
                    help="benchmark configuration: d = headline (Llama-3-8B DP-SGD); a = CPU MLP plumbing; b = GPT-2-small "
                         "DP-SGD; c = Llama-3.2-1B DP-FTRL (BLT); e = OLMoE-1B-7B")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.config == "a":
        run_config_a(args)
        return
    preset = {"b": dict(model="gpt2-small", seq=1024, batch=1024, sigma=0.8), "c": dict(model="llama3.2-1b", seq=2048, batch=512,
              sigma=1.0, blt_buffers=4), "e": dict(model="olmoe-1b-7b", seq=2048, batch=512, sigma=1.0)}.get(args.config, {})
    for k, v in preset.items():
        if getattr(args, k) == ap.get_default(k):
            setattr(args, k, v)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    from opake_b200.models.config import PRESETS
    from opake_b200.ops import _lib
    from opake_b200.parallel import comm
    from opake_b200.parallel.engine import EngineConfig, ShardedDPEngine

    rank, world, local = comm.init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    mcfg = PRESETS[args.model]()
    if args.batch % world:
        raise SystemExit("logical batch must divide evenly over the ranks")
    b_local = args.batch // world
    blt = {}
    if args.blt_buffers:
        k = args.blt_buffers
        blt = dict(blt_decay=tuple(1.0 - 0.5 ** (i + 1) * 0.9 for i in range(k)), blt_scale=tuple(0.5 / k for _ in range(k)),
                   noise_stream_tag="opake.dpftrl.mf_gaussian")
    shard = args.shard if args.shard != "auto" else ("full" if world > 1 else "state")
    ecfg = EngineConfig(clip_norm=1.0, noise_multiplier=args.sigma, logical_batch=args.batch, lr=3e-4, weight_decay=0.01,
                        noise_bias_correction=True, master_weights=False, use_cuda_graph=not args.no_graph,
                        attn_impl=args.attn, seed=1234, accumulate_group=args.group,
                        shard_params=shard in ("params", "full"), shard_sums=shard == "full",
                        expert_parallel=bool(mcfg.n_experts) and world > 1, seq_len=args.seq,
                        comm_backend=args.comm, **blt)
    eng = ShardedDPEngine(mcfg, ecfg, dev)

    tok = _zipf_tokens(b_local, args.seq, mcfg.vocab_size, seed=1000 + rank)
    labels = torch.roll(tok, -1, dims=1).clone()
    labels[:, -1] = -100
    labels[:, : args.seq // 4] = -100                       # SFT mask: no loss on the first 25 % of each sequence
    tok_h, lab_h = tok.pin_memory(), labels.pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    last_loss = None
    for _ in range(args.warmup):
        last_loss = eng.step(tok_h, lab_h).item()
    # ---- ONE timed region: every step copies its inputs from pinned host memory (per example, inside the engine) and
    # reads its loss back to the host; CUDA events and the wall clock bracket the same steps, max over ranks.
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = _lib.LAUNCHES[0] + eng.graph_kernel_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        last_loss = eng.step(tok_h, lab_h).item()
    e1.record()
    barrier()
    e2e_s = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1)
    launches = _lib.LAUNCHES[0] + eng.graph_kernel_launches - launches0
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    tokens = args.batch * args.seq * args.steps
    value = tokens / (dev_ms / 1e3)
    e2e_value = tokens / (e2e_ms / 1e3)
    if rank == 0:
        print(json.dumps({
            "metric": "DP tokens/sec/box (max over ranks), Llama-3-8B FSDP DP-SGD" if args.config == "d" else
                      f"DP tokens/sec/box (max over ranks), config {args.config}: {mcfg.name}",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic Zipf(1.1) tokens, random-init weights", "impl": "ours",
            "config": {"model": mcfg.name, "layers": mcfg.n_layers, "global_batch": args.batch, "seq_len": args.seq,
                       "parallelism": f"fsdp{world} " + {
                           "state": "(optimizer moments sharded; bf16 parameters and fp32 sums replicated, reduce-scatter by peer "
                                    "loads and all-gather by peer stores inside the fused step kernel)",
                           "params": "(optimizer moments and parameters sharded: each tensor has one owner and is fetched inside "
                                     "the first forward GEMMs after a step; fp32 sums replicated)",
                           "full": "(full shard: optimizer moments, parameters and fp32 sums; parameters fetched inside the first "
                                   "forward GEMMs after a step, accumulation groups reduce-scattered by reductions over NVLink)",
                       }[shard] + f"; gathered bf16 parameters cached across the {b_local} accumulation micro-steps",
                       "shard": shard, "step_collectives": args.comm, "expert_parallel": f"ep{world}" if (mcfg.n_experts and world > 1) else None,
                       "clip_norm": 1.0, "noise_multiplier": args.sigma, "optimizer": "adamw-bc", "sft_mask": "first 25%",
                       "mechanism": f"dp-ftrl blt x{args.blt_buffers}" if args.blt_buffers else "dp-sgd gaussian",
                       "per_example_microbatch": 1, "cuda_graph": not args.no_graph,
                       "accumulate_group": getattr(eng, "group", None),
                       "device_memory_in_use_gib": round((lambda f, t: (t - f) / 2 ** 30)(*torch.cuda.mem_get_info(dev)), 1),
                       "l2_policy": "inputs larger than L2: every example streams all bf16 weights and a full-size bf16 gradient, "
                                    f"{2 * eng.layout.total / 2 ** 30:.1f} GiB each, far beyond the 126 MB L2",
                       "final_loss_per_example": last_loss / b_local},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": int(2 * b_local * args.seq * 4), "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
