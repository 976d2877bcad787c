"""Conversion of Hugging Face ``TrainingArguments`` (or any object / mapping with those attribute names) into this
package's ``TrainingArguments`` (packages/opake-transformers/src/opake/api/transformers/trainer/_hf_convert.py:125-540,
_convert.py:22-224). Gradient accumulation collapses into the logical batch (DP has no notion of it: a step is one
noise addition), ``max_grad_norm`` becomes the clipping norm, optimizer spellings collapse to the DP optimizers,
Liger flags turn the fused kernels on. DeepSpeed is rejected; ``fsdp`` maps onto the native sharded engine."""
from __future__ import annotations

import dataclasses
import warnings
from typing import Any, Mapping

from ..base.exceptions import ConfigurationError

__all__ = ["convert_hf_training_arguments", "DROPPED_FIELDS"]

# fields with no meaning under DP training; a non-default value is reported once and ignored
DROPPED_FIELDS = ("gradient_accumulation_steps", "max_grad_norm", "fp16", "fp16_full_eval", "half_precision_backend",
                  "auto_find_batch_size", "group_by_length", "length_column_name", "neftune_noise_alpha",
                  "optim_target_modules", "batch_eval_metrics", "eval_use_gather_object", "use_liger_kernel",
                  "liger_kernel_config", "accelerator_config", "parallelism_config", "ddp_find_unused_parameters",
                  "ddp_bucket_cap_mb", "ddp_broadcast_buffers", "past_index", "jit_mode_eval", "use_legacy_prediction_loop")
_OPTIM_ALIASES = {"adamw_torch": "adamw", "adamw_torch_fused": "adamw", "adamw_hf": "adamw", "adamw_apex_fused": "adamw",
                  "adamw_anyprecision": "adamw", "adamw_8bit": "adamw", "paged_adamw_32bit": "adamw",
                  "sgd": "sgd", "adagrad": "adagrad", "adafactor": "adafactor", "rmsprop": "rmsprop", "lion_32bit": "lion",
                  "ademamix": "ademamix", "schedule_free_adamw": "schedule_free", "schedule_free_sgd": "schedule_free"}


def _get(src: Any, name: str, default=None):
    if isinstance(src, Mapping):
        return src.get(name, default)
    return getattr(src, name, default)


def _enum_value(v):
    return getattr(v, "value", v)


def convert_hf_training_arguments(hf_args: Any, cls, **dp_overrides: Any):
    if _get(hf_args, "deepspeed"):
        raise ConfigurationError("DeepSpeed configurations cannot be converted: per-example clipping needs control of "
                                 "the backward pass. Use fsdp=True for sharded DP training.")
    names = {f.name for f in dataclasses.fields(cls)}
    out: dict[str, Any] = {}
    for name in names:
        v = _get(hf_args, name, None)
        if v is not None:
            out[name] = _enum_value(v)
    # scheduler field is called lr_scheduler_type upstream
    sched = _get(hf_args, "lr_scheduler_type")
    if sched is not None:
        out["lr_scheduler"] = {"cosine_with_min_lr": "cosine", "reduce_lr_on_plateau": "constant",
                               "warmup_stable_decay": "warmup_stable_decay"}.get(_enum_value(sched), _enum_value(sched))
    # logical batch = per-device batch x accumulation
    accum = int(_get(hf_args, "gradient_accumulation_steps", 1) or 1)
    bs = int(_get(hf_args, "per_device_train_batch_size", 8) or 8)
    out["per_device_train_batch_size"] = bs * accum
    if accum > 1 and "microbatch_size" not in dp_overrides:
        out["microbatch_size"] = bs
    optim = _enum_value(_get(hf_args, "optim", "adamw"))
    if optim is not None:
        key = str(optim).lower()
        out["optim"] = _OPTIM_ALIASES.get(key, key)
    ratio = _get(hf_args, "warmup_ratio", 0.0) or 0.0
    if ratio and not _get(hf_args, "warmup_steps", 0):
        out["warmup_steps"] = float(ratio)
    mgn = _get(hf_args, "max_grad_norm")
    if mgn is not None and mgn > 0 and "clipping_norm" not in dp_overrides:
        out["clipping_norm"] = float(mgn)
    if _get(hf_args, "use_liger_kernel"):
        out["use_performance_kernels"] = True
    if _get(hf_args, "fp16"):
        warnings.warn("fp16 is not supported for DP training (no loss scaling under clipping); using bf16", stacklevel=2)
        out["bf16"] = True
    fsdp = _get(hf_args, "fsdp")
    if fsdp:
        out["fsdp"] = True
    for name in DROPPED_FIELDS:
        v = _get(hf_args, name)
        if v not in (None, False, 0, 0.0, "", [], {}, 1, 1.0) and name not in ("gradient_accumulation_steps", "max_grad_norm",
                                                                              "use_liger_kernel", "fp16"):
            warnings.warn(f"TrainingArguments.{name}={v!r} has no effect under DP training and is dropped", stacklevel=2)
    out.update(dp_overrides)
    return cls(**{k: v for k, v in out.items() if k in names})
