"""Command line of the framework: ``python -m opake_b200.cli <command> [--preset NAME] [options]``.

Commands

* ``dpsgd``    DP-SGD training (Poisson or k-out-of-t sampling, Gaussian noise, fixed / AUTO-S / adaptive clipping)
* ``dpftrl``   DP-FTRL training (matrix-factorisation noise: identity, band-MF, BLT, BISR, BSR, lambda-CGD)
* ``sft``      supervised fine-tuning with completion masks (``SFTTrainer``)
* ``dpo``      preference optimisation (``DPOTrainer``, 17 loss heads)
* ``account``  privacy arithmetic without training: epsilon of a schedule, or the noise multiplier for a target epsilon
* ``families`` the registered Hugging Face model families and what is patched for each

The option vocabulary and the preset mechanism follow the reference's training script (``examples/train_dpsgd.py:354-980``:
``--preset`` fills defaults, explicit flags win). Data is synthetic unless ``--text-file`` / ``--jsonl-file`` names a
local file (byte-level tokens); nothing is downloaded. Models are the native decoder presets (``--model-name``) or a
local Hugging Face checkpoint directory (``--hf-model``), which is patched with ``apply_model_patches`` or lowered to the
native runtime when its family supports it. Under ``torchrun`` the native engine shards optimizer state, parameters
and gradient sums (``--shard``) or, for mixture-of-experts presets, the experts (``--expert-parallel``).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
from typing import Any

PRESETS: dict[str, dict[str, Any]] = {
    # quick functional check on a CPU
    "smoke": dict(model_name="tiny-llama", num_train_samples=256, num_eval_samples=32, max_seq_len=64, batch_size=16, num_epochs=1,
                  log_steps=2, eval_steps=0, target_epsilon=8.0, learning_rate=1e-3, dtype="float32", audit=False),
    # the five benchmark configurations (shapes, batch and noise of each)
    "gpt2-small-dpsgd": dict(model_name="gpt2-small", max_seq_len=1024, batch_size=1024, noise_multiplier=0.8, clipping_norm=1.0,
                             learning_rate=3e-4, optimizer="adamw-bc", num_train_samples=1_000_000, dtype="bfloat16"),
    "llama1b-dpftrl-blt": dict(model_name="llama3.2-1b", max_seq_len=2048, batch_size=512, noise_multiplier=1.0, mechanism="mf_blt",
                               max_buffers=4, optimizer="adamw-bc", shard="full", dtype="bfloat16"),
    "llama8b-dpsgd-fsdp": dict(model_name="llama3-8b", max_seq_len=2048, batch_size=256, noise_multiplier=0.9, clipping_norm=1.0,
                               optimizer="adamw-bc", shard="full", dtype="bfloat16", microbatch_size=1),
    "olmoe-dpsgd-ep": dict(model_name="olmoe-1b-7b", max_seq_len=2048, batch_size=512, noise_multiplier=1.0, clipping_norm=1.0,
                           optimizer="adamw-bc", expert_parallel=True, dtype="bfloat16"),
}

_MECHANISM_FLAGS = {"mf_band": ("bands",), "mf_blt": ("max_buffers",), "mf_bisr": ("bandwidth",),
                    "mf_bsr": ("bandwidth", "alpha", "beta"), "mf_lambda_cgd": ("lambda_",)}


def _add_training_flags(p: argparse.ArgumentParser, *, ftrl: bool = False) -> None:
    g = p.add_argument_group("model / data")
    g.add_argument("--preset", choices=sorted(PRESETS), default=None, help="fills defaults; explicit flags win")
    g.add_argument("--model-name", default=None, help="native preset: tiny-llama, gpt2-small, llama3.2-1b, llama3-8b, olmoe-1b-7b")
    g.add_argument("--hf-model", default=None, help="local Hugging Face checkpoint directory (patched, or lowered when supported)")
    g.add_argument("--text-file", default=None, help="local text file, byte-level tokens, cut into sequences")
    g.add_argument("--jsonl-file", default=None, help="local JSON-lines file; --dataset-text-field names the text column")
    g.add_argument("--dataset-text-field", default="text")
    g.add_argument("--num-train-samples", type=int, default=None)
    g.add_argument("--num-eval-samples", type=int, default=None)
    g.add_argument("--max-seq-len", type=int, default=None)
    g.add_argument("--dtype", choices=("float32", "bfloat16"), default=None)
    g.add_argument("--cpu", action="store_true")
    g = p.add_argument_group("optimisation")
    g.add_argument("--batch-size", type=int, default=None, help="expected logical batch (all ranks)")
    g.add_argument("--eval-batch-size", type=int, default=None)
    g.add_argument("--microbatch-size", type=int, default=None, help="0 = whole batch under one vmap")
    g.add_argument("--num-epochs", type=float, default=None)
    g.add_argument("--stop-at-step", type=int, default=None)
    g.add_argument("--learning-rate", type=float, default=None)
    g.add_argument("--lr-schedule", default=None)
    g.add_argument("--lr-warmup-steps", type=float, default=None)
    g.add_argument("--lr-min-ratio", type=float, default=None)
    g.add_argument("--optimizer", default=None)
    g.add_argument("--noise-bias-correction", action=argparse.BooleanOptionalAction, default=None)
    g.add_argument("--weight-decay", type=float, default=None)
    g.add_argument("--gradient-checkpointing", action="store_true")
    g.add_argument("--activation-offloading", action="store_true")
    g.add_argument("--kernel-patches", action=argparse.BooleanOptionalAction, default=True)
    g.add_argument("--shard", choices=("none", "state", "params", "full"), default=None,
                   help="what the native engine shards over the ranks")
    g.add_argument("--expert-parallel", action=argparse.BooleanOptionalAction, default=None)
    g.add_argument("--log-steps", type=int, default=None)
    g.add_argument("--eval-steps", type=int, default=None)
    g.add_argument("--output-dir", default="trainer_output")
    g.add_argument("--resume", default=None)
    g.add_argument("--seed", type=int, default=42)
    g = p.add_argument_group("privacy")
    g.add_argument("--target-epsilon", type=float, default=None)
    g.add_argument("--target-delta", type=float, default=None)
    g.add_argument("--noise-multiplier", type=float, default=None)
    g.add_argument("--calibration-min", type=float, default=None)
    g.add_argument("--calibration-max", type=float, default=None)
    g.add_argument("--calibration-tolerance", type=float, default=None)
    g.add_argument("--clipping-mode", choices=("fixed", "auto", "adaptive"), default=None)
    g.add_argument("--clipping-norm", type=float, default=None)
    g.add_argument("--per-group-clipping", default=None, help='JSON {"pattern": norm, ...} of path substrings')
    g.add_argument("--target-clipping-rate", type=float, default=None, help="adaptive clipping: target quantile")
    g.add_argument("--clipping-norm-max", type=float, default=None)
    g.add_argument("--auto-clipping-gamma", type=float, default=None)
    g.add_argument("--second-moment", action="store_true", help="privatise squared gradients for the optimizer's second moment")
    g.add_argument("--sampler", default=None)
    g.add_argument("--truncated-batch-size", type=int, default=None)
    g.add_argument("--k", type=int, default=None, help="k-out-of-t sampling: participations per example")
    g.add_argument("--allocation", choices=("block", "total"), default=None)
    if ftrl:
        g.add_argument("--mechanism", choices=("mf_identity", "mf_band", "mf_blt", "mf_bisr", "mf_bsr", "mf_lambda_cgd"), default=None)
        g.add_argument("--bands", type=int, default=None)
        g.add_argument("--max-buffers", type=int, default=None)
        g.add_argument("--bandwidth", type=int, default=None)
        g.add_argument("--alpha", type=float, default=None)
        g.add_argument("--beta", type=float, default=None)
        g.add_argument("--lambda", dest="lambda_", type=float, default=None)
    g = p.add_argument_group("auditing")
    g.add_argument("--audit", action=argparse.BooleanOptionalAction, default=None, help="one-run privacy audit with canaries")
    g.add_argument("--audit-canaries", type=int, default=64)
    g.add_argument("--audit-method", choices=("eps_delta", "gdp"), default="eps_delta")


_DEFAULTS = dict(model_name="tiny-llama", num_train_samples=2048, num_eval_samples=0, max_seq_len=64, dtype=None, batch_size=64,
                 eval_batch_size=None, microbatch_size=None, num_epochs=1.0, stop_at_step=None, learning_rate=1e-3,
                 lr_schedule="cosine", lr_warmup_steps=0, lr_min_ratio=None, optimizer="adamw-bc", noise_bias_correction=None,
                 weight_decay=0.0, shard=None, expert_parallel=None, log_steps=5, eval_steps=0, target_epsilon=None,
                 target_delta=None, noise_multiplier=None, clipping_mode="fixed", clipping_norm=1.0, sampler="auto", audit=False,
                 mechanism="mf_band", bands=None, max_buffers=None, bandwidth=None, alpha=None, beta=None, lambda_=None)


def resolve(args: argparse.Namespace) -> argparse.Namespace:
    """Explicit flags, then the preset, then the built-in defaults."""
    preset = PRESETS.get(args.preset or "", {})
    for name, default in _DEFAULTS.items():
        if getattr(args, name, None) is None:
            setattr(args, name, preset.get(name, default))
    for name, value in preset.items():
        if not hasattr(args, name) or getattr(args, name) is None:
            setattr(args, name, value)
    if args.microbatch_size == 0:
        args.microbatch_size = None
    if args.target_epsilon is None and args.noise_multiplier is None:
        args.target_epsilon = 8.0
    return args


# ----------------------------------------------------------------------------------------------------------- data
def _byte_sequences(text: bytes, seq: int, limit: int):
    import torch

    ids = torch.frombuffer(bytearray(text), dtype=torch.uint8).to(torch.int64)
    n = min(limit, ids.numel() // seq)
    if n < 1:
        raise SystemExit(f"the file holds fewer than {seq} bytes")
    return ids[: n * seq].view(n, seq)


class _TokenRows:
    """Rows of token ids as a map-style dataset with a completion mask over the last 75 % of each sequence."""

    def __init__(self, rows):
        self.rows = rows
        self._fingerprint = f"rows-{tuple(rows.shape)}-{int(rows.sum())}"

    def __len__(self):
        return self.rows.shape[0]

    def __getitem__(self, i):
        ids = self.rows[i].tolist()
        cut = len(ids) // 4
        return {"input_ids": ids, "completion_mask": [0] * cut + [1] * (len(ids) - cut)}


def build_datasets(a, vocab: int):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples"))
    n_train, n_eval = a.num_train_samples, a.num_eval_samples or 0
    if a.text_file or a.jsonl_file:
        if a.text_file:
            raw = open(a.text_file, "rb").read()
        else:
            with open(a.jsonl_file, encoding="utf-8") as f:
                raw = "\n".join(json.loads(line)[a.dataset_text_field] for line in f if line.strip()).encode()
        if vocab < 256:
            raise SystemExit("byte-level data needs a vocabulary of at least 256 entries")
        rows = _byte_sequences(raw, a.max_seq_len, n_train + n_eval)
        n_eval = min(n_eval, rows.shape[0] // 10)
        return _TokenRows(rows[: rows.shape[0] - n_eval]), (_TokenRows(rows[rows.shape[0] - n_eval :]) if n_eval else None)
    from .alignment.data import SyntheticLM

    train = SyntheticLM(n_train, vocab, a.max_seq_len, a.seed)
    return train, (SyntheticLM(n_eval, vocab, a.max_seq_len, a.seed + 1) if n_eval else None)


# ----------------------------------------------------------------------------------------------------------- model
def build_model(a):
    import torch

    from .models.config import PRESETS as MODEL_PRESETS
    from .models.native import NativeCausalLM

    cuda = torch.cuda.is_available() and not a.cpu
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, None: torch.bfloat16 if cuda else torch.float32}[a.dtype]
    if a.hf_model:
        from transformers import AutoModelForCausalLM

        from . import patches

        hf = AutoModelForCausalLM.from_pretrained(a.hf_model, torch_dtype=dtype)
        spec = patches.family_of(hf)
        if spec is not None and spec.native and cuda:
            return patches.to_native(hf, dtype=dtype, device="cuda"), "native (lowered from Hugging Face weights)"
        report = patches.apply_model_patches(hf, kernels=bool(a.kernel_patches and cuda))
        return hf.to("cuda" if cuda else "cpu"), f"vmap(grad) over the patched Hugging Face model {report}"
    if a.model_name not in MODEL_PRESETS:
        raise SystemExit(f"unknown --model-name {a.model_name!r}; choose from {sorted(MODEL_PRESETS)}")
    cfg = MODEL_PRESETS[a.model_name]()
    if a.max_seq_len > cfg.max_seq:
        from dataclasses import replace

        cfg = replace(cfg, max_seq=a.max_seq_len)
    return NativeCausalLM(cfg, dtype=dtype, device="cuda" if cuda else None), ("native sm_100a runtime" if cuda else "portable path (CPU)")


def runtime_report(a, how: str) -> None:
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    print(f"[opake_b200] model: {a.hf_model or a.model_name} ({how})")
    print(f"[opake_b200] device: {'cuda' if torch.cuda.is_available() and not a.cpu else 'cpu'}, ranks: {world}, "
          f"shard: {a.shard or ('full' if world > 1 else 'none')}, expert parallel: {bool(a.expert_parallel)}")
    print(f"[opake_b200] batch {a.batch_size} x {a.max_seq_len} tokens, microbatch {a.microbatch_size}, optimizer {a.optimizer}, "
          f"clipping {a.clipping_mode} C={a.clipping_norm}")


# ----------------------------------------------------------------------------------------------------------- arguments
def training_arguments(a, cls, *, mechanism: str = "gaussian", mechanism_kwargs: dict | None = None, extra: dict | None = None):
    steps_per_epoch = max(1, a.num_train_samples // a.batch_size)
    max_steps = a.stop_at_step if a.stop_at_step else max(1, int(math.ceil(a.num_epochs * steps_per_epoch)))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    optim = a.optimizer
    if a.noise_bias_correction and optim in ("adamw", "adam"):
        optim = "adamw-bc"
    clipping_kwargs: dict[str, Any] = {}
    if a.clipping_mode == "adaptive":
        clipping_kwargs = {k: v for k, v in (("target_quantile", a.target_clipping_rate), ("clipping_norm_max", a.clipping_norm_max)) if v is not None}
    if a.clipping_mode == "auto" and a.auto_clipping_gamma is not None:
        clipping_kwargs["gamma"] = a.auto_clipping_gamma
    if a.second_moment:
        clipping_kwargs["second_moment"] = True
    norm: Any = a.clipping_norm
    if a.per_group_clipping:
        norm = json.loads(a.per_group_clipping)
    sampling_kwargs = {k: v for k, v in (("truncated_batch_size", a.truncated_batch_size), ("k", a.k), ("allocation", a.allocation)) if v is not None}
    calib = {k: v for k, v in (("param_min", a.calibration_min), ("param_max", a.calibration_max), ("tolerance", a.calibration_tolerance)) if v is not None}
    sched_kwargs = {"min_lr_ratio": a.lr_min_ratio} if a.lr_min_ratio is not None else {}
    kw = dict(output_dir=a.output_dir, per_device_train_batch_size=max(1, a.batch_size // world),
              per_device_eval_batch_size=a.eval_batch_size or max(1, (a.microbatch_size or 8)), microbatch_size=a.microbatch_size,
              max_steps=max_steps, learning_rate=a.learning_rate, optim=optim, lr_scheduler=a.lr_schedule, lr_scheduler_kwargs=sched_kwargs,
              warmup_steps=a.lr_warmup_steps, weight_decay=a.weight_decay, seed=a.seed, use_cpu=a.cpu, clipping_norm=norm,
              clipping_mode=a.clipping_mode, clipping_kwargs=clipping_kwargs, logging_steps=max(1, a.log_steps), save_strategy="no",
              eval_strategy="steps" if a.eval_steps else "no", eval_steps=a.eval_steps or None, log_level="info",
              privacy_target_delta=a.target_delta, resume_from_checkpoint=a.resume, privacy_noise_mechanism=mechanism,
              privacy_noise_mechanism_kwargs=mechanism_kwargs or {}, sampling_mode=a.sampler, sampling_kwargs=sampling_kwargs,
              noise_calibration_kwargs=calib, gradient_checkpointing=a.gradient_checkpointing,
              activation_offloading=a.activation_offloading, use_performance_kernels=bool(a.kernel_patches),
              fsdp=(a.shard or ("full" if world > 1 else "none")) != "none", expert_parallel=world if a.expert_parallel else 1,
              bf16=a.dtype == "bfloat16")
    if a.noise_multiplier is not None:
        kw["privacy_noise_multiplier"] = a.noise_multiplier
    else:
        kw["privacy_target_epsilon"] = a.target_epsilon
    kw.update(extra or {})
    fields = {f.name for f in __import__("dataclasses").fields(cls)}
    return cls(**{k: v for k, v in kw.items() if k in fields})


def _finish(trainer, out, a) -> dict:
    metrics = {k: (round(v, 6) if isinstance(v, float) else v) for k, v in out.metrics.items()}
    if a.audit:
        metrics.update(run_audit(trainer, a))
    print(json.dumps(metrics, default=str))
    return metrics


def run_audit(trainer, a) -> dict:
    """One-run audit (Steinke et al.): canaries are included by coin flips, scored by their loss after training, and the
    guesses are turned into a lower bound on epsilon."""
    from . import auditing
    from .engine.random import fold_in, key

    ds = trainer.train_dataset
    flips = auditing.coin_flip(ds, num_canaries=min(a.audit_canaries, len(ds)), key=fold_in(key(a.seed), "audit"))
    scores = trainer.audit_loss_scores(flips) if hasattr(trainer, "audit_loss_scores") else None
    if scores is None:
        return {"audit": "skipped: this trainer exposes no per-example loss for scoring"}
    est = auditing.one_run(scores, coin_flip=flips)
    method = est.eps_delta() if a.audit_method == "eps_delta" else est.gdp()
    return {"audit_epsilon_lower_bound": float(method.epsilon_at(trainer._rt.get("target_delta") or 1e-5))}


# ----------------------------------------------------------------------------------------------------------- commands
def cmd_train(a, kind: str) -> dict:
    from .alignment.sft import language_modeling_collator
    from .transformers import DPTrainer, SFTConfig, SFTTrainer, TrainingArguments

    a = resolve(a)
    model, how = build_model(a)
    runtime_report(a, how)
    vocab = model.cfg.vocab_size if hasattr(model, "cfg") else model.config.vocab_size
    train, evald = build_datasets(a, vocab)
    mech, mkw = "gaussian", {}
    if kind == "dpftrl":
        mech = a.mechanism
        mkw = {f: getattr(a, f) for f in _MECHANISM_FLAGS.get(mech, ()) if getattr(a, f, None) is not None}
    if kind == "sft":
        args = training_arguments(a, SFTConfig, mechanism=mech, mechanism_kwargs=mkw, extra={"max_length": a.max_seq_len})
        trainer = SFTTrainer(model, args, train_dataset=train, eval_dataset=evald)
    else:
        args = training_arguments(a, TrainingArguments, mechanism=mech, mechanism_kwargs=mkw)
        trainer = DPTrainer(model, args, data_collator=language_modeling_collator(0, a.max_seq_len), train_dataset=train,
                            eval_dataset=evald)
    return _finish(trainer, trainer.train(), a)


def cmd_dpo(a) -> dict:
    from .alignment.data import SyntheticPreferences
    from .transformers import DPOConfig, DPOTrainer

    a = resolve(a)
    model, how = build_model(a)
    runtime_report(a, how)
    vocab = model.cfg.vocab_size if hasattr(model, "cfg") else model.config.vocab_size
    half = max(4, a.max_seq_len // 2)
    data = SyntheticPreferences(a.num_train_samples, vocab, half, half, a.seed)
    args = training_arguments(a, DPOConfig, extra={"loss_type": a.loss_type, "beta": a.dpo_beta, "max_length": 2 * half,
                                                   "native_engine": False})
    trainer = DPOTrainer(model, None, args, train_dataset=data)
    return _finish(trainer, trainer.train(), a)


def cmd_account(a) -> dict:
    from . import accounting as acc
    from .dpsgd import accounting as sgd_acc

    q = a.batch_size / a.dataset_size
    delta = a.target_delta if a.target_delta is not None else 1.0 / a.dataset_size ** 1.1

    def process(nm):
        step = sgd_acc.poisson(sgd_acc.gaussian(nm), q, truncated_batch_size=a.truncated_batch_size,
                               dataset_size=a.dataset_size if a.truncated_batch_size else None)
        return step * a.steps

    if a.noise_multiplier is not None:
        out = {"noise_multiplier": a.noise_multiplier, "epsilon": process(a.noise_multiplier).epsilon_at(delta), "delta": delta}
    else:
        res = acc.calibrate(acc.epsilon_budget(a.target_epsilon, delta=delta), process, a.calibration_min, a.calibration_max)
        out = {"noise_multiplier": res.param, "epsilon": res.achieved, "delta": delta}
    out.update(sample_rate=q, steps=a.steps)
    print(json.dumps(out))
    return out


def cmd_families(_a) -> dict:
    from .patches import FAMILIES

    rows = {n: {"native": s.native, "moe": s.moe, "sliding_window": s.sliding_window, "norm_offset": s.norm_offset,
                "softcap": s.softcap, "act": s.act, "notes": s.notes} for n, s in sorted(FAMILIES.items())}
    print(json.dumps(rows, indent=1))
    return rows


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="opake_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = p.add_subparsers(dest="command", required=True)
    for name in ("dpsgd", "dpftrl", "sft"):
        _add_training_flags(sub.add_parser(name, help=f"{name} training"), ftrl=name == "dpftrl")
    d = sub.add_parser("dpo", help="preference optimisation")
    _add_training_flags(d)
    d.add_argument("--loss-type", default="sigmoid")
    d.add_argument("--dpo-beta", type=float, default=0.1)
    c = sub.add_parser("account", help="epsilon of a DP-SGD schedule, or the noise multiplier for a target epsilon")
    c.add_argument("--dataset-size", type=int, required=True)
    c.add_argument("--batch-size", type=int, required=True)
    c.add_argument("--steps", type=int, required=True)
    c.add_argument("--noise-multiplier", type=float, default=None)
    c.add_argument("--target-epsilon", type=float, default=8.0)
    c.add_argument("--target-delta", type=float, default=None)
    c.add_argument("--truncated-batch-size", type=int, default=None)
    c.add_argument("--calibration-min", type=float, default=0.3)
    c.add_argument("--calibration-max", type=float, default=50.0)
    sub.add_parser("families", help="registered model families")
    return p


def main(argv: list[str] | None = None):
    a = build_parser().parse_args(argv)
    if a.command in ("dpsgd", "dpftrl", "sft"):
        return cmd_train(a, a.command)
    if a.command == "dpo":
        return cmd_dpo(a)
    if a.command == "account":
        return cmd_account(a)
    return cmd_families(a)


if __name__ == "__main__":
    main()
