"""Shared pieces of the example command lines: synthetic token datasets (no network needed) and argument groups."""
from __future__ import annotations

import argparse

import torch


from opake_b200.alignment.data import SyntheticLM, SyntheticPreferences  # noqa: E402,F401


def add_common(p: argparse.ArgumentParser) -> None:
    g = p.add_argument_group("model / data")
    g.add_argument("--model", default="tiny-llama", help="preset name: tiny-llama, llama3.2-1b, llama3-8b, gpt2-small")
    g.add_argument("--dataset-size", type=int, default=2048)
    g.add_argument("--seq-len", type=int, default=64)
    g.add_argument("--cpu", action="store_true")
    g = p.add_argument_group("optimisation")
    g.add_argument("--batch-size", type=int, default=64)
    g.add_argument("--microbatch-size", type=int, default=None)
    g.add_argument("--max-steps", type=int, default=20)
    g.add_argument("--lr", type=float, default=1e-3)
    g.add_argument("--optim", default="adamw-bc")
    g.add_argument("--lr-scheduler", default="cosine")
    g.add_argument("--warmup-steps", type=float, default=0)
    g.add_argument("--output-dir", default="trainer_output")
    g.add_argument("--resume", default=None)
    g.add_argument("--seed", type=int, default=42)
    g = p.add_argument_group("privacy")
    g.add_argument("--epsilon", type=float, default=None)
    g.add_argument("--delta", type=float, default=None)
    g.add_argument("--noise-multiplier", type=float, default=None)
    g.add_argument("--clipping-norm", type=float, default=1.0)
    g.add_argument("--clipping-mode", default="fixed", choices=("fixed", "auto", "adaptive"))


def preset(name: str):
    from opake_b200.models import config as C
    table = {"tiny-llama": C.tiny_llama, "llama3.2-1b": C.llama32_1b, "llama3-8b": C.llama3_8b, "gpt2-small": C.gpt2_small,
             "olmoe-1b-7b": C.olmoe_1b_7b}
    return table[name]()


def training_kwargs(a) -> dict:
    kw = dict(output_dir=a.output_dir, per_device_train_batch_size=a.batch_size, microbatch_size=a.microbatch_size,
              max_steps=a.max_steps, learning_rate=a.lr, optim=a.optim, lr_scheduler=a.lr_scheduler, warmup_steps=a.warmup_steps,
              seed=a.seed, use_cpu=a.cpu, clipping_norm=a.clipping_norm, clipping_mode=a.clipping_mode, logging_steps=5,
              save_strategy="no", log_level="info", privacy_target_delta=a.delta, resume_from_checkpoint=a.resume)
    if a.noise_multiplier is not None:
        kw["privacy_noise_multiplier"] = a.noise_multiplier
    else:
        kw["privacy_target_epsilon"] = a.epsilon if a.epsilon is not None else 8.0
    return kw
