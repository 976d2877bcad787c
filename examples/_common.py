"""Shared pieces of the example command lines: synthetic token datasets (no network needed) and argument groups."""
from __future__ import annotations

import argparse

import torch


class SyntheticLM(torch.utils.data.Dataset):
    """Zipf-distributed token sequences with a completion mask on the last 75 % of every sequence."""

    def __init__(self, n: int, vocab: int, seq: int, seed: int = 0):
        self.n, self.vocab, self.seq, self.seed = n, vocab, seq, seed
        ranks = torch.arange(1, vocab + 1, dtype=torch.float64)
        self.p = (ranks ** -1.1 / (ranks ** -1.1).sum()).float()
        self._fingerprint = f"synthetic-lm-{n}-{vocab}-{seq}-{seed}"

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        ids = torch.multinomial(self.p, self.seq, replacement=True, generator=g).tolist()
        cut = self.seq // 4
        return {"input_ids": ids, "completion_mask": [0] * cut + [1] * (self.seq - cut)}


class SyntheticPreferences(torch.utils.data.Dataset):
    def __init__(self, n: int, vocab: int, prompt: int = 16, completion: int = 16, seed: int = 0):
        self.n, self.vocab, self.prompt, self.completion, self.seed = n, vocab, prompt, completion, seed
        self._fingerprint = f"synthetic-pref-{n}-{vocab}-{prompt}-{completion}-{seed}"

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        p, c, r = (torch.randint(0, self.vocab, (k,), generator=g).tolist() for k in (self.prompt, self.completion, self.completion))
        return {"chosen_input_ids": p + c, "rejected_input_ids": p + r, "chosen_completion_mask": [0] * len(p) + [1] * len(c),
                "rejected_completion_mask": [0] * len(p) + [1] * len(r)}


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
