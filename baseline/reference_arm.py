"""Reference arm of the benchmark: the unmodified reference framework on the headline configuration.

Runs the reference's own public API and stock code path, exactly as its ``examples/train_dpsgd.py`` does
(``examples/train_dpsgd.py:1145-1149,1356-1385,1529-1538,1870-1898``):

    transformers ``LlamaForCausalLM`` -> ``opake.patches.apply_model_patches`` -> ``opake.functional.make_functional``
    -> ``opake.dpsgd.clipping.clipped_grad(microbatch_size=...)`` -> ``opake.distributed.gradients.sum_gradients_`` (N > 1)
    -> ``opake.dpsgd.noise.gaussian_noise`` -> ``opake.optimizers.adamw(noise_bias_correction=True)`` -> ``torchopt.apply_updates``

Nothing of this repository's package (models, kernels, engine) is imported here. The reference packages are the
unmodified sources installed under ``baseline/_ref``; ``optree`` and ``torchopt`` (absent from the image) are the
stand-ins under ``baseline/third_party_shims`` and are declared in the JSON line.

The reference draws its Gaussian noise on the CPU, leaf by leaf, and copies it to the device
(``opake-dpsgd/src/opake/api/dpsgd/noise/_gaussian.py:188-204``), so one optimizer step of an 8-billion-parameter model takes
minutes. The arm therefore works against a wall-clock budget: it runs the requested warm-up and timed steps while they
fit, and otherwise as many timed steps as fit (at least one) after the warm-up; the JSON line reports the counts it
actually used next to the requested ones.
"""
from __future__ import annotations

import glob
import inspect
import json
import os
import sys
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")   # allocator setting only; the reference is untouched
HERE = os.path.dirname(os.path.abspath(__file__))
T_PROCESS_START = time.perf_counter()


def _say(obj: dict) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(obj), flush=True)


def _paths() -> list[str]:
    return [os.path.join(HERE, "third_party_shims")] + sorted(glob.glob(os.path.join(HERE, "_ref", "opake-*")))


def _zipf_tokens(n_seq: int, seq: int, vocab: int, seed: int):
    import numpy as np
    import torch

    rng = np.random.default_rng(seed)
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    p = ranks ** -1.1
    p /= p.sum()
    cdf = np.cumsum(p)
    u = rng.random((n_seq, seq))
    return torch.from_numpy(np.searchsorted(cdf, u).clip(0, vocab - 1).astype(np.int64))


MODEL_SHAPES = {
    # name: (vocab, hidden, ffn, layers, heads, kv heads, rope theta)
    "llama3-8b": (128256, 4096, 14336, 32, 32, 8, 500000.0),
    "llama3.2-1b": (128256, 2048, 8192, 16, 32, 8, 500000.0),
    "tiny": (512, 64, 128, 2, 4, 2, 500000.0),
}


def run(args) -> None:
    pkgs = _paths()
    if len(pkgs) < 5:
        _say({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference packages (install each reference sub-project with pip --no-deps --target baseline/_ref/opake-<name>)"})
        return
    sys.path[:0] = pkgs
    try:
        import torch
        import torch.distributed as dist
        import torchopt
        from transformers import LlamaConfig, LlamaForCausalLM

        from opake.distributed.gradients import sum_gradients_
        from opake.dpsgd.clipping import clipped_grad
        from opake.dpsgd.noise import gaussian_noise
        from opake.functional import make_functional
        from opake.optimizers import adamw
        from opake.patches import apply_model_patches, apply_runtime_patches
        from opake.random import key
    except Exception as exc:  # noqa: BLE001 - any import failure makes the arm unavailable
        _say({"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"[:400]})
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and args.model != "tiny-cpu"
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if use_cuda else "gloo", device_id=dev if use_cuda else None)

    model_name = "tiny" if args.model == "tiny-cpu" else args.model
    vocab, hidden, ffn, layers, heads, kv, theta = MODEL_SHAPES[model_name]
    if getattr(args, "layers", 0):
        layers = args.layers
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=kv, max_position_embeddings=max(args.seq, 2048), rope_theta=theta, tie_word_embeddings=False,
                      attention_dropout=0.0, use_cache=False)
    dtype = torch.bfloat16 if use_cuda else torch.float32
    torch.manual_seed(1234)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with dev:
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    model.train()

    budget_s = float(os.environ.get("OPK_REF_BUDGET_S", "640"))
    b_local = args.batch // world
    kernels_mode = "triton kernels + fused linear-CE" if use_cuda else "eager"
    apply_runtime_patches()
    try:
        apply_model_patches(model, kernels=use_cuda, fused_linear_cross_entropy=use_cuda)
    except Exception as exc:  # noqa: BLE001 - fall back to the reference's own eager baseline switch
        kernels_mode = f"eager (kernel patches failed: {type(exc).__name__})"
        apply_model_patches(model, kernels=False, fused_linear_cross_entropy=False)
    fmodel, trainable, frozen = make_functional(model, disable_autograd_tracking=True, partition_trainable=True)
    try:
        fwd_params = inspect.signature(model.forward).parameters
        marker = use_cuda and "loss_only" in fwd_params
    except (TypeError, ValueError):
        marker = False

    def per_example_loss(tr, input_ids, labels):
        extra = {"loss_only": True} if marker else {}
        out = fmodel({**frozen, **tr}, input_ids.unsqueeze(0), labels=labels.unsqueeze(0), **extra)
        return out.loss

    noise_fn, noise_state = gaussian_noise(noise_multiplier=args.sigma, key=key(1234))
    opt = adamw(lr=3e-4, weight_decay=0.01, noise_bias_correction=True)
    opt_state = opt.init(trainable)

    tok = _zipf_tokens(b_local, args.seq, vocab, seed=1000 + rank)
    labels = tok.clone()
    labels[:, : args.seq // 4] = -100                       # SFT mask: no loss on the first 25 % (the model shifts labels itself)
    tok_h = tok.pin_memory() if use_cuda else tok
    lab_h = labels.pin_memory() if use_cuda else labels

    def sync():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize(dev)

    state = {"trainable": trainable, "opt": opt_state, "noise": noise_state}

    def build(mb):
        return clipped_grad(per_example_loss, argnums=0, batch_argnums=(1, 2), clipping_norm=1.0, normalize_by=args.batch,
                            microbatch_size=mb, return_aux=True)

    def one_step(grad_fn, clip_state):
        ids = tok_h.to(dev, non_blocking=True)
        lab = lab_h.to(dev, non_blocking=True)
        (grads, aux), clip_state = grad_fn(state["trainable"], ids, lab, state=clip_state)
        if world > 1:
            sum_gradients_(grads)
        noisy, state["noise"] = noise_fn(grads, state["noise"])
        upd, state["opt"] = opt.update(noisy, state["opt"], params=state["trainable"])
        state["trainable"] = torchopt.apply_updates(state["trainable"], upd)
        return float(aux.loss_values.sum()), clip_state                        # device -> host read of the step's summed per-example loss

    # ---- warm-up with step-down: a step that runs out of memory (the optimizer state and the fp32 clip-sum buffer appear
    # during the first steps) moves on to the next smaller microbatch, as the reference's DPTrainer does on OOM, and the
    # warm-up starts over. Every rank takes the same decision.
    candidates = [int(x) for x in os.environ.get("OPK_REF_MICROBATCH", "2,1").split(",")]
    note = lambda msg: print(f"[reference arm rank {rank}] {msg}", file=sys.stderr, flush=True)  # noqa: E731
    grad_fn = clip_state = None
    mb_used, oom_msg, step_s, warm_done = None, "", None, 0
    ci = 0
    while ci < len(candidates) and warm_done < max(1, args.warmup):
        mb = candidates[ci]
        if grad_fn is None:
            grad_fn, clip_state = build(mb)
        failed = 0
        try:
            sync()
            t0 = time.perf_counter()
            _, clip_state = one_step(grad_fn, clip_state)
            if use_cuda:
                torch.cuda.synchronize(dev)
            step_s = time.perf_counter() - t0
        except torch.OutOfMemoryError as exc:
            failed, oom_msg = 1, str(exc)[:300]
        flag = torch.tensor([failed], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag.item()):
            note(f"out of memory at microbatch {mb}: {oom_msg[:120]}")
            grad_fn = clip_state = None
            warm_done, ci = 0, ci + 1
            if use_cuda:
                torch.cuda.empty_cache()
            continue
        mb_used, warm_done = mb, warm_done + 1
        note(f"warm-up step {warm_done} at microbatch {mb}: {step_s:.1f} s")
        # stop warming up early when the remaining budget only holds one timed step
        elapsed = time.perf_counter() - T_PROCESS_START
        stop = torch.tensor([1 if budget_s - elapsed < 2.2 * step_s else 0], device=dev)
        if world > 1:
            dist.broadcast(stop, 0)
        if int(stop.item()):
            break
    if mb_used is None or grad_fn is None:
        _say({"impl": "reference", "unavailable": f"out of memory at microbatch sizes {candidates} on the headline configuration: {oom_msg}"})
        return
    elapsed = time.perf_counter() - T_PROCESS_START
    plan = torch.tensor([max(1, min(args.steps, int(max(0.0, budget_s - elapsed) // max(step_s, 1e-3))))], device=dev)
    if world > 1:
        dist.broadcast(plan, 0)
    steps = int(plan.item())
    first_step_s = step_s

    sync()
    if use_cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    last = 0.0
    for k in range(steps):
        last, clip_state = one_step(grad_fn, clip_state)
        note(f"timed step {k + 1} of {steps} issued")
    if use_cuda:
        e1.record()
    sync()
    wall_ms = (time.perf_counter() - t0) * 1e3
    dev_ms = e0.elapsed_time(e1) if use_cuda else wall_ms
    t = torch.tensor([dev_ms, wall_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = t.tolist()
    tokens = args.batch * args.seq * steps
    peak_gb = torch.cuda.max_memory_allocated(dev) / 2 ** 30 if use_cuda else None
    _say({
        "metric": "DP tokens/sec/box (max over ranks), Llama-3-8B FSDP DP-SGD" if model_name == "llama3-8b" else
                  f"DP tokens/sec/box (max over ranks), {model_name}",
        "impl": "reference", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warm_done, "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": dev_ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if use_cuda else "fp32", "data": "synthetic Zipf(1.1) tokens, random-init weights",
        "config": {"model": model_name, "layers": layers, "global_batch": args.batch, "seq_len": args.seq,
                   "parallelism": f"ddp{world} (the reference has no FSDP; per-leaf NCCL all-reduce of the clipped sum)",
                   "clip_norm": 1.0, "noise_multiplier": args.sigma, "optimizer": "adamw-bc", "sft_mask": "first 25%",
                   "per_example_microbatch": mb_used, "model_patches": kernels_mode, "fused_lce_marker": bool(marker),
                   "noise": "CPU torch.Generator, leaf by leaf, copied to the device (reference stock path)",
                   "wall_budget_s": budget_s, "first_step_s": first_step_s, "peak_memory_gib": peak_gb,
                   "l2_policy": "inputs larger than L2: every step streams 16 GB of bf16 weights",
                   "final_loss_per_example": last / max(b_local, 1)},
        "third_party_stand_ins": ["optree", "torchopt"],
        "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "ms_per_step": wall_ms / steps,
                "h2d_bytes_per_step": int(2 * b_local * args.seq * 8), "d2h_bytes_per_step": 4},
        "gpu_launches": 0,
    })
    if world > 1:
        dist.destroy_process_group()
