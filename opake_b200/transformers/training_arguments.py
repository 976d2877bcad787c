"""``TrainingArguments``: one dataclass holding every knob of ``DPTrainer`` (packages/opake-transformers/src/opake/api/
transformers/trainer/_training_arguments.py:298-620; pairing tables :186-212, mechanism defaults :253-264).

The Hugging Face field names are kept so that existing launch scripts carry over; the DP fields follow. New here:
``fsdp`` (shard gradient sums, optimizer state and parameters over ranks with the fused reduce-scatter /
AdamW / all-gather step), ``expert_parallel`` (ranks that share a MoE layer's experts) and ``native_engine``
(run supported decoder families on the hand-written sm_100a runtime instead of ``vmap(grad)``).
"""
from __future__ import annotations

import dataclasses
import json
import math
from dataclasses import dataclass, field
from typing import Any

from ..base.exceptions import ConfigurationError

__all__ = ["TrainingArguments", "DEFAULT_SAMPLING", "ALLOWED_SAMPLING", "MECHANISM_DEFAULTS", "default_delta"]

NOISE_MECHANISMS = ("gaussian", "mf_identity", "mf_band", "mf_blt", "mf_bisr", "mf_bsr", "mf_lambda_cgd")
CLIPPING_MODES = ("fixed", "adaptive", "auto")
# default sampler for every noise mechanism and the overrides that keep the privacy analysis valid
DEFAULT_SAMPLING = {"gaussian": "poisson", "mf_identity": "poisson", "mf_band": "cyclic_poisson", "mf_blt": "balls_in_bins",
                    "mf_bisr": "balls_in_bins", "mf_bsr": "balls_in_bins", "mf_lambda_cgd": "balls_in_bins"}
ALLOWED_SAMPLING = {"gaussian": {"poisson", "k_out_of_t"}, "mf_identity": {"poisson", "balls_in_bins"},
                    "mf_band": {"cyclic_poisson", "b_min_sep"}, "mf_blt": {"balls_in_bins"}, "mf_bisr": {"balls_in_bins"},
                    "mf_bsr": {"balls_in_bins"}, "mf_lambda_cgd": {"balls_in_bins"}}
MECHANISM_DEFAULTS: dict[str, dict[str, Any]] = {
    "gaussian": {}, "mf_identity": {}, "mf_band": {"bands": 16}, "mf_blt": {"max_buffers": 10},
    "mf_bisr": {"bandwidth": 4}, "mf_bsr": {"bandwidth": 8, "alpha": 1.0, "beta": 0.9}, "mf_lambda_cgd": {"lambda_": 0.5},
}
_STRATEGIES = ("no", "steps", "epoch")
_SCHEDULERS = ("linear", "cosine", "cosine_with_restarts", "polynomial", "constant", "constant_with_warmup",
               "inverse_sqrt", "warmup_stable_decay", "cosine_with_min_lr", "cosine_warmup_with_min_lr", "exponential",
               "one_minus_sqrt")


def default_delta(dataset_size: int) -> float:
    """delta = 1 / N^1.1, the default privacy target when none is given."""
    return 1.0 / (max(int(dataset_size), 2) ** 1.1)


@dataclass
class TrainingArguments:
    # ---- output / batch / optimisation (Hugging Face names)
    output_dir: str = "trainer_output"
    overwrite_output_dir: bool = False
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int = 8
    eval_accumulation_steps: int | None = None
    eval_delay: float = 0.0
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    optim: str = "adamw"
    optim_args: str | dict | None = None
    lr_scheduler: str = "linear"
    lr_scheduler_kwargs: dict = field(default_factory=dict)
    warmup_steps: int | float = 0
    num_train_epochs: float = 3.0
    max_steps: int = -1
    # ---- logging / saving
    log_level: str = "passive"
    log_level_replica: str = "warning"
    log_on_each_node: bool = True
    logging_dir: str | None = None
    logging_strategy: str = "steps"
    logging_first_step: bool = False
    logging_steps: float = 500
    save_strategy: str = "steps"
    save_steps: float = 500
    save_total_limit: int | None = None
    save_safetensors: bool = True
    save_on_each_node: bool = False
    save_only_model: bool = False
    restore_callback_states_from_checkpoint: bool = False
    # ---- reproducibility / device
    seed: int = 42
    data_seed: int | None = None
    full_determinism: bool = False
    use_cpu: bool = False
    use_mps_device: bool = False
    bf16: bool = False
    bf16_full_eval: bool = False
    tf32: bool | None = None
    local_rank: int = -1
    ddp_backend: str | None = None
    ddp_timeout: int = 1800
    # ---- evaluation
    eval_strategy: str = "no"
    eval_steps: float | None = None
    eval_on_start: bool = False
    eval_do_concat_batches: bool = True
    prediction_loss_only: bool = False
    include_for_metrics: list = field(default_factory=list)
    average_tokens_across_devices: bool = True
    metric_for_best_model: str | None = None
    greater_is_better: bool | None = None
    load_best_model_at_end: bool = False
    ignore_data_skip: bool = False
    # ---- data loading
    dataloader_num_workers: int = 0
    dataloader_persistent_workers: bool = False
    dataloader_pin_memory: bool = True
    dataloader_prefetch_factor: int | None = None
    dataloader_multiprocessing_context: str | None = None
    dataloader_in_order: bool = True
    dataloader_drop_last: bool = False
    remove_unused_columns: bool = True
    torch_empty_cache_steps: int | None = None
    label_names: list | None = None
    label_smoothing_factor: float = 0.0
    # ---- reporting / hub
    report_to: str | list | None = "none"
    disable_tqdm: bool | None = None
    run_name: str | None = None
    project: str | None = None
    trackio_space_id: str | None = None
    push_to_hub: bool = False
    hub_model_id: str | None = None
    hub_strategy: str = "every_save"
    hub_token: str | None = None
    hub_private_repo: bool | None = None
    hub_always_push: bool = False
    hub_revision: str | None = None
    # ---- compilation / memory
    torch_compile: bool = False
    torch_compile_backend: str | None = None
    torch_compile_mode: str | None = None
    gradient_checkpointing: bool = False
    gradient_checkpointing_kwargs: dict | None = None
    skip_memory_metrics: bool = True
    include_tokens_per_second: bool = False
    include_num_input_tokens_seen: bool = False
    debug: str | list = ""
    resume_from_checkpoint: str | bool | None = None
    # ---- differential privacy
    microbatch_size: int | None = None
    auto_find_microbatch_size: bool = False
    clipping_norm: float | dict | str = 1.0
    cuda_graphs: int = 0
    use_performance_kernels: bool = False
    performance_kernels_config: dict | None = None
    use_compat_patches: bool = True
    activation_offloading: bool = False
    privacy_target_epsilon: float | None = None
    privacy_target_delta: float | None = None
    privacy_accounting: bool = True
    clipping_mode: str = "fixed"
    clipping_kwargs: dict = field(default_factory=dict)
    privacy_noise_mechanism: str = "gaussian"
    privacy_noise_multiplier: float | None = None
    privacy_noise_mechanism_kwargs: dict = field(default_factory=dict)
    sampling_mode: str = "auto"
    sampling_kwargs: dict = field(default_factory=dict)
    noise_calibration_kwargs: dict = field(default_factory=dict)
    enable_jit_checkpoint: bool = False
    # ---- parallelism beyond plain data parallel (not present in the reference trainer)
    fsdp: bool = False
    expert_parallel: int = 1
    native_engine: str | bool = "auto"          # "auto" | True | False

    # ------------------------------------------------------------------------------------------- validation
    def __post_init__(self):
        if self.per_device_train_batch_size < 1 or self.per_device_eval_batch_size < 1:
            raise ConfigurationError("per-device batch sizes must be positive")
        for name in ("logging_strategy", "save_strategy", "eval_strategy"):
            v = getattr(self, name)
            v = getattr(v, "value", v)
            if v not in _STRATEGIES:
                raise ConfigurationError(f"{name} must be one of {_STRATEGIES}, got {v!r}")
            setattr(self, name, v)
        self.lr_scheduler = getattr(self.lr_scheduler, "value", self.lr_scheduler)
        if callable(self.lr_scheduler) and not isinstance(self.lr_scheduler, str):
            pass        # a schedule recipe (step -> lr); the scheduler factory checks that no warm-up / kwargs come with it
        elif self.lr_scheduler not in _SCHEDULERS:
            raise ConfigurationError(f"lr_scheduler must be one of {_SCHEDULERS}, got {self.lr_scheduler!r}")
        if self.clipping_mode not in CLIPPING_MODES:
            raise ConfigurationError(f"clipping_mode must be one of {CLIPPING_MODES}, got {self.clipping_mode!r}")
        if self.privacy_noise_mechanism not in NOISE_MECHANISMS:
            raise ConfigurationError(f"privacy_noise_mechanism must be one of {NOISE_MECHANISMS}, got "
                                     f"{self.privacy_noise_mechanism!r}")
        if self.sampling_mode != "auto" and self.sampling_mode not in ALLOWED_SAMPLING[self.privacy_noise_mechanism]:
            raise ConfigurationError(f"sampling_mode {self.sampling_mode!r} is not valid for noise mechanism "
                                     f"{self.privacy_noise_mechanism!r}; allowed: "
                                     f"{sorted(ALLOWED_SAMPLING[self.privacy_noise_mechanism])}")
        # both given: the noise is fixed and training STOPS when the accountant reaches the target (stop-at-epsilon)
        if self.privacy_target_epsilon is not None and self.privacy_noise_multiplier is not None and self.privacy_noise_multiplier == 0.0:
            raise ConfigurationError("privacy_noise_multiplier=0.0 is the non-private path; privacy_target_epsilon is "
                                     "meaningless there")
        if self.privacy_target_epsilon is not None and self.privacy_target_epsilon <= 0:
            raise ConfigurationError("privacy_target_epsilon must be positive")
        if self.privacy_target_delta is not None and not 0 < self.privacy_target_delta < 1:
            raise ConfigurationError("privacy_target_delta must be in (0, 1)")
        if isinstance(self.clipping_norm, (int, float)) and not isinstance(self.clipping_norm, bool):
            if not (self.clipping_norm > 0 and math.isfinite(self.clipping_norm)):
                raise ConfigurationError("clipping_norm must be positive and finite")
        if self.microbatch_size is not None and self.microbatch_size < 1:
            raise ConfigurationError("microbatch_size must be positive")
        if self.load_best_model_at_end and self.eval_strategy == "no":
            raise ConfigurationError("load_best_model_at_end requires an eval_strategy")
        if self.load_best_model_at_end and self.metric_for_best_model is None:
            self.metric_for_best_model = "loss"
        if self.metric_for_best_model is not None and self.greater_is_better is None:
            self.greater_is_better = not self.metric_for_best_model.endswith("loss")
        if self.expert_parallel < 1:
            raise ConfigurationError("expert_parallel must be >= 1")
        if self.torch_compile:
            raise ConfigurationError("torch_compile is not supported: the hot path is hand-written CUDA, captured in "
                                     "CUDA graphs (set cuda_graphs instead)")
        if isinstance(self.report_to, str):
            self.report_to = [] if self.report_to in ("none", "") else [self.report_to]
        elif self.report_to is None:
            self.report_to = []
        if self.disable_tqdm is None:
            self.disable_tqdm = True
        if isinstance(self.optim_args, str):
            self.optim_args = dict(kv.split("=", 1) for kv in self.optim_args.replace(" ", "").split(",") if kv)

    # ------------------------------------------------------------------------------------------- derived values
    @property
    def world_size(self) -> int:
        from ..engine import distributed as D
        return D.get_world_size()

    @property
    def train_batch_size(self) -> int:
        """Expected logical batch over all ranks (the quantity the sampling rate is derived from)."""
        return self.per_device_train_batch_size * max(1, self.world_size)

    @property
    def resolved_sampling_mode(self) -> str:
        return DEFAULT_SAMPLING[self.privacy_noise_mechanism] if self.sampling_mode == "auto" else self.sampling_mode

    @property
    def resolved_mechanism_kwargs(self) -> dict:
        return {**MECHANISM_DEFAULTS[self.privacy_noise_mechanism], **self.privacy_noise_mechanism_kwargs}

    @property
    def is_dpftrl(self) -> bool:
        return self.privacy_noise_mechanism.startswith("mf_")

    def target_delta(self, dataset_size: int) -> float:
        return self.privacy_target_delta if self.privacy_target_delta is not None else default_delta(dataset_size)

    def resolve_interval(self, value: float | None, total_steps: int, fallback: float | None = None) -> int | None:
        """``logging_steps`` / ``save_steps`` / ``eval_steps`` below 1 are fractions of the total number of steps."""
        v = fallback if value is None else value
        if v is None:
            return None
        return max(1, int(math.ceil(v * total_steps))) if v < 1 else int(v)

    def resolve_warmup(self, total_steps: int) -> int:
        w = self.warmup_steps
        return int(math.ceil(w * total_steps)) if 0 < w < 1 else int(w)

    # ------------------------------------------------------------------------------------------- (de)serialisation
    def to_dict(self) -> dict:
        d = dataclasses.asdict(self)
        d.pop("hub_token", None)
        return d

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True, default=str)

    @classmethod
    def from_dict(cls, d: dict) -> "TrainingArguments":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    @classmethod
    def from_hf(cls, hf_args: Any, **dp_overrides: Any) -> "TrainingArguments":
        from .hf_convert import convert_hf_training_arguments
        return convert_hf_training_arguments(hf_args, cls, **dp_overrides)
