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

__all__ = ["convert_hf_training_arguments", "convert_trl_config", "ConversionReport", "DROPPED_FIELDS", "REJECTED_FIELDS"]

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


# values that cannot be honoured and would silently change what is trained: the conversion refuses them
REJECTED_FIELDS = {
    "deepspeed": "DeepSpeed owns the backward pass and the optimizer; per-example clipping needs both (use fsdp=True)",
    "packing": "packed sequences mix several examples in one row, which breaks per-example clipping",
    "padding_free": "padding-free batches concatenate examples, which breaks per-example clipping",
    "use_liger_loss": "the Liger fused loss has no per-example form; use_performance_kernels selects this package's kernels",
}
# alternative spellings (TRL / older Hugging Face releases) -> field of this package
_RENAMES = {"lr_scheduler_type": "lr_scheduler", "max_seq_length": "max_length", "evaluation_strategy": "eval_strategy",
            "activation_offloading": "activation_offloading", "torch_empty_cache_steps": "torch_empty_cache_steps",
            "dataset_num_proc": None, "dataset_kwargs": None, "model_init_kwargs": None}


@dataclasses.dataclass
class ConversionReport:
    """What happened to every field of the source arguments: copied under its own name, renamed / collapsed into
    another field, dropped (no meaning under DP training) or overridden by an explicit DP keyword."""

    copied: list = dataclasses.field(default_factory=list)
    renamed: dict = dataclasses.field(default_factory=dict)
    dropped: dict = dataclasses.field(default_factory=dict)
    overridden: list = dataclasses.field(default_factory=list)


def _get(src: Any, name: str, default=None):
    if isinstance(src, Mapping):
        return src.get(name, default)
    return getattr(src, name, default)


def _enum_value(v):
    return getattr(v, "value", v)


def convert_hf_training_arguments(hf_args: Any, cls, *, return_report: bool = False, **dp_overrides: Any):
    for bad, why in REJECTED_FIELDS.items():
        if _get(hf_args, bad):
            raise ConfigurationError(f"{bad}={_get(hf_args, bad)!r} cannot be converted: {why}")
    report = ConversionReport()
    names = {f.name for f in dataclasses.fields(cls)}
    out: dict[str, Any] = {}
    for name in names:
        v = _get(hf_args, name, None)
        if v is not None:
            out[name] = _enum_value(v)
            report.copied.append(name)
    for old, new in _RENAMES.items():
        v = _get(hf_args, old)
        if v is None or new is None or new not in names or old == new:
            continue
        out[new] = _enum_value(v)
        report.renamed[old] = new
    # non-reentrant layer checkpointing is the only form that composes with vmap(grad): the reentrant request is rewritten
    gck = _get(hf_args, "gradient_checkpointing_kwargs")
    if isinstance(gck, Mapping) and gck.get("use_reentrant"):
        out["gradient_checkpointing_kwargs"] = {k: v for k, v in gck.items() if k != "use_reentrant"}
        report.renamed["gradient_checkpointing_kwargs.use_reentrant"] = "ignored (functional checkpointing)"
    if _get(hf_args, "torch_compile"):
        report.dropped["torch_compile"] = "the hot path is hand-written kernels and CUDA graphs"
        out["torch_compile"] = False
    # scheduler field is called lr_scheduler_type upstream
    sched = _get(hf_args, "lr_scheduler_type")
    if sched is not None:
        out["lr_scheduler"] = {"cosine_with_min_lr": "cosine", "reduce_lr_on_plateau": "constant",
                               "warmup_stable_decay": "warmup_stable_decay"}.get(_enum_value(sched), _enum_value(sched))
    # logical batch = per-device batch x accumulation
    accum = int(_get(hf_args, "gradient_accumulation_steps", 1) or 1)
    bs = int(_get(hf_args, "per_device_train_batch_size", 8) or 8)
    out["per_device_train_batch_size"] = bs * accum
    if accum > 1:
        report.renamed["gradient_accumulation_steps"] = "per_device_train_batch_size (logical batch) + microbatch_size"
        if "microbatch_size" not in dp_overrides:
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
        report.renamed["max_grad_norm"] = "clipping_norm (per example)"
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
        if (v is True or v not in (None, False, 0, 0.0, "", [], {}, 1, 1.0)) and name not in ("gradient_accumulation_steps", "max_grad_norm",
                                                                              "use_liger_kernel", "fp16"):
            warnings.warn(f"TrainingArguments.{name}={v!r} has no effect under DP training and is dropped", stacklevel=2)
            report.dropped[name] = "no effect under DP training"
    report.overridden = sorted(k for k in dp_overrides if k in out)
    out.update(dp_overrides)
    built = cls(**{k: v for k, v in out.items() if k in names})
    return (built, report) if return_report else built


def convert_trl_config(trl_config: Any, cls, *, return_report: bool = False, **dp_overrides: Any):
    """TRL ``SFTConfig`` / ``DPOConfig`` (objects or mappings) -> this package's trainer configs. On top of the Hugging
    Face rules: ``max_seq_length`` is the older name of ``max_length``; packing and padding-free batches are refused;
    ``loss_type`` lists and ``beta`` / ``label_smoothing`` / ``reference_free`` carry over by name."""
    return convert_hf_training_arguments(trl_config, cls, return_report=return_report, **dp_overrides)
