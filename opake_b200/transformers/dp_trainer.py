"""``DPTrainer``: a Hugging-Face-shaped training loop for differentially private training (packages/opake-
transformers/src/opake/api/transformers/trainer/_dp_trainer.py:484-6061; call stack of ``train`` :1045-2233,
``training_step`` :2290-2505, ``evaluate`` :3245, ``predict`` :3321, checkpointing :5317-5461).

It does not subclass the Hugging Face trainer. One step is: privacy-sampled batch -> per-example clipped gradient
sum -> (all-reduce) -> calibrated noise -> DP-aware optimizer -> accountant. Two execution paths share the loop:

* the generic path works for any ``nn.Module``: ``make_functional`` + ``vmap(grad)`` clipping from
  ``opake_b200.dpsgd`` / ``dpftrl``, pytree optimizers, explicit all-reduce of the clipped sum;
* the native path (``NativeCausalLM`` models on CUDA) hands the step to ``ShardedDPEngine``: per-example CUDA graphs
  of hand-written sm_100a kernels and one fused reduce-scatter + noise + AdamW + all-gather kernel over peer memory.
"""
from __future__ import annotations

import json
import math
import os
import shutil
import time
import warnings
from typing import Any, Callable

import numpy as np
import torch
from torch import nn
from torch.utils.data import DataLoader

from .. import accounting as acc
from ..base.exceptions import CheckpointError, ConfigurationError, OperationError, PrivacyBudgetError
from ..base.serialization import from_state_dict, state_dict
from ..dpsgd import clipping as clip_api
from ..dpsgd import noise as sgd_noise
from ..engine import distributed as D
from ..engine.functional import empty_collate, make_functional
from ..engine.profiling import step_perf
from ..engine.pytree import tree_map
from ..engine.random import RngKey, fold_in, key as make_key
from ..optimizers import apply_updates
from . import checkpoint as ckpt
from . import dpftrl as mf
from .callback import CallbackHandler, PrinterCallback, TrainerCallback, reporting_callbacks
from .distributed import DDPState, checkpoint_barrier, resolve_ddp_state
from .eval import (EvaluationResult, EvaluationTelemetry, PredictionAccumulator, PredictionOutput, resolve_eval_num_samples,
                   speed_metrics, with_metric_prefix)
from .optim import build_optimizer
from .precision import autocast_context
from .scheduler import build_lr_schedule
from .state import DPTrainerState, TrainerControl
from .training_arguments import TrainingArguments

__all__ = ["DPTrainer", "TrainOutput"]

_SAMPLER_TAG = "opake.transformers.sampler"
_NOISE_TAG = "opake.transformers.noise"
_IGNORE_DATA_SKIP_TAG = "opake.transformers.ignore_data_skip"


class TrainOutput(tuple):
    """``(global_step, training_loss, metrics)`` with attribute access."""

    def __new__(cls, global_step, training_loss, metrics):
        return super().__new__(cls, (global_step, training_loss, metrics))

    global_step = property(lambda s: s[0])
    training_loss = property(lambda s: s[1])
    metrics = property(lambda s: s[2])


def _is_oom(e: BaseException) -> bool:
    return isinstance(e, torch.cuda.OutOfMemoryError) or (isinstance(e, RuntimeError) and "out of memory" in str(e).lower())


def _to_device(batch, device):
    if isinstance(batch, torch.Tensor):
        return batch.to(device, non_blocking=True)
    if isinstance(batch, dict):
        return {k: _to_device(v, device) for k, v in batch.items()}
    if isinstance(batch, (list, tuple)):
        return type(batch)(_to_device(v, device) for v in batch)
    return batch


def _batch_len(batch) -> int:
    if isinstance(batch, torch.Tensor):
        return batch.shape[0]
    if isinstance(batch, dict):
        for v in batch.values():
            n = _batch_len(v)
            if n >= 0:
                return n
        return -1
    if isinstance(batch, (list, tuple)) and batch:
        return _batch_len(batch[0])
    return -1


def _rank_local_sampler_state(saved_state, template_sampler, world_size: int):
    """Re-key a sampler snapshot onto this rank's own stream (``trainer/_dp_trainer.py:216-252`` of the reference).

    Only the main rank writes the snapshot, so it carries the main rank's rank-folded stream key and the length of the
    main rank's data shard. Installing it verbatim would give every rank the same Poisson coins (perfectly correlated
    inclusion across shards, which the amplification analysis does not allow) and fail the length check whenever the
    shards differ in size. Under DDP the key and the shard length therefore come from this rank's freshly built
    sampler and only the cursor (and the sampler's hyper-parameters) from the snapshot."""
    if world_size <= 1 or "key_seed" not in saved_state:
        return saved_state
    key = getattr(template_sampler, "_stream_key", None)
    if key is None:
        raise CheckpointError(f"sampler snapshot carries a stream key but {type(template_sampler).__name__} exposes none; "
                              "cannot restore a rank-local sampling stream under DDP")
    local = dict(saved_state)
    local["key_seed"] = int(key.seed)
    if "key_impl" in local:
        local["key_impl"] = str(key.impl)
    own = template_sampler.state_dict()
    for name in ("num_samples",):
        if name in local and name in own:
            local[name] = own[name]
    return local


def predict_stop_step(prefix_process, step_process, *, target_epsilon: float, delta: float, k0: int, horizon: int) -> int | None:
    """First accounted step in ``(k0, horizon]`` at which epsilon reaches ``target_epsilon``, or ``None`` (not reached
    within the horizon, or the epsilon sequence failed the boundary check). After ``k`` steps the accountant holds
    ``prefix | step_process * (k - k0)``, so a monotone epsilon(k) is bisected with about ``log2(horizon)`` evaluations
    (packages/opake-transformers/src/opake/api/transformers/trainer/_dp_trainer.py:350-410)."""
    remaining = horizon - k0
    if remaining < 1:
        return None
    cache: dict[int, float] = {}

    def eps(j: int) -> float:
        if j not in cache:
            proc = step_process * j if prefix_process is None else prefix_process | (step_process * j)
            cache[j] = float(proc.epsilon_at(delta))
        return cache[j]

    if eps(remaining) < target_epsilon:
        return None
    lo, hi = 1, remaining
    while lo < hi:
        mid = (lo + hi) // 2
        if eps(mid) >= target_epsilon:
            hi = mid
        else:
            lo = mid + 1
    if eps(lo) < target_epsilon or (lo > 1 and eps(lo - 1) >= target_epsilon):
        warnings.warn(f"stop-at-epsilon: epsilon is not monotone near step {k0 + lo}; checking at log boundaries instead",
                      stacklevel=2)
        return None
    return k0 + lo


class DPTrainer:
    def __init__(self, model: nn.Module | None = None, args: TrainingArguments | None = None, data_collator: Callable | None = None,
                 train_dataset=None, eval_dataset=None, processing_class=None, compute_loss_func: Callable | None = None,
                 compute_metrics: Callable | None = None, callbacks: list | None = None, optimizers: tuple = (None, None),
                 optimizer_cls_and_kwargs: tuple | None = None, preprocess_logits_for_metrics: Callable | None = None):
        if model is None:
            raise ConfigurationError("DPTrainer needs a model")
        self.args = args if args is not None else TrainingArguments()
        self.model = model
        self.data_collator = data_collator
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.processing_class = processing_class
        self.compute_loss_func, self.compute_metrics = compute_loss_func, compute_metrics
        self.preprocess_logits_for_metrics = preprocess_logits_for_metrics
        self._user_optimizer, self._user_scheduler = optimizers
        self._optimizer_cls_and_kwargs = optimizer_cls_and_kwargs
        self.device = self._resolve_device()
        self.ddp: DDPState = resolve_ddp_state(self.args.ddp_backend, self.device, self.args.ddp_timeout)
        self.state = DPTrainerState(is_world_process_zero=self.ddp.is_main, is_local_process_zero=self.ddp.local_rank == 0,
                                    world_size=self.ddp.world_size, ddp_backend=self.ddp.backend)
        self.control = TrainerControl()
        self.hub_model_id = None
        default_cbs: list = [] if self.args.disable_tqdm and not self.args.logging_first_step and self.args.log_level == "passive" else []
        self.callback_handler = CallbackHandler(default_cbs + reporting_callbacks(self.args.report_to) + list(callbacks or []),
                                                model=model, processing_class=processing_class)
        if self.args.log_level in ("info", "debug"):
            self.callback_handler.add_callback(PrinterCallback())
        self.accountant: acc.Accountant | None = None
        self.optimizer = None
        self.lr_scheduler: Callable[[int], float] | None = None
        self._native = None            # ShardedDPEngine when the native path is active
        self._rt: dict[str, Any] = {}  # runtime objects of the generic path (params, states, fns)
        self._microbatch = self.args.microbatch_size
        if self.args.full_determinism:
            from ..engine.random import set_reproducible_pytorch_seed
            set_reproducible_pytorch_seed(self.args.seed)
        else:
            torch.manual_seed(self.args.seed)
        if self.args.tf32 is not None and torch.cuda.is_available():
            torch.backends.cuda.matmul.allow_tf32 = bool(self.args.tf32)
        self.control = self.callback_handler.call_event("on_init_end", self.args, self.state, self.control)

    # ------------------------------------------------------------------------------------------- small helpers
    def _resolve_device(self) -> torch.device:
        if self.args.use_cpu or not torch.cuda.is_available():
            return torch.device("cpu")
        local = int(os.environ.get("LOCAL_RANK", max(self.args.local_rank, 0)))
        torch.cuda.set_device(local)
        return torch.device("cuda", local)

    def add_callback(self, cb):
        self.callback_handler.add_callback(cb)

    def pop_callback(self, cb):
        return self.callback_handler.pop_callback(cb)

    def remove_callback(self, cb):
        self.callback_handler.remove_callback(cb)

    def is_world_process_zero(self) -> bool:
        return self.ddp.is_main

    def log(self, logs: dict) -> None:
        logs = dict(logs)
        if self.state.epoch is not None:
            logs["epoch"] = round(self.state.epoch, 4)
        self.state.log_history.append({**logs, "step": self.state.global_step})
        self.control = self.callback_handler.call_event("on_log", self.args, self.state, self.control, logs=logs)

    def _use_native(self) -> bool:
        from ..models.native import NativeCausalLM
        want = self.args.native_engine
        ok = isinstance(self.model, NativeCausalLM) and self.device.type == "cuda"
        if want is True and not ok:
            raise ConfigurationError("native_engine=True needs a NativeCausalLM model and a CUDA device")
        if want is False:
            return False
        if ok and (self.args.is_dpftrl and self.args.privacy_noise_mechanism not in ("mf_blt", "mf_identity", "mf_band", "mf_bsr")):
            if want is True:
                raise ConfigurationError("the native engine implements Gaussian, buffered-linear-Toeplitz, band-MF and "
                                         "banded-square-root noise")
            return False
        if ok and self.args.clipping_mode == "adaptive":
            return False
        return ok

    def is_local_process_zero(self) -> bool:
        return self.ddp.local_rank == 0

    @property
    def label_names(self) -> list:
        return list(self.args.label_names or ["labels"])

    # ------------------------------------------------------------------------------------------- loss seam
    def compute_per_example_loss_and_metrics(self, call: Callable, params, inputs: dict):
        """``(loss, {name: per-example tensor})`` of ONE example: the seam for objectives that report per-example
        telemetry (preference rewards, margins). The values ride the clipping transform's ``loss_aux`` channel, are summed
        over ranks, averaged per logged step and aggregated in the evaluation loop. The default has no telemetry and
        delegates to :meth:`compute_per_example_loss`; overriding THIS method turns the aux channel on."""
        return self.compute_per_example_loss(call, params, inputs), {}

    def _overrides_metrics_seam(self) -> bool:
        return type(self).compute_per_example_loss_and_metrics is not DPTrainer.compute_per_example_loss_and_metrics

    def compute_per_example_loss(self, call: Callable, params, inputs: dict) -> torch.Tensor:
        """Loss of ONE example. ``call(params, **inputs)`` runs the model on a batch of one; subclasses override this
        to change the objective (the SFT / DPO trainers do)."""
        outputs = call(params, **inputs)
        labels = inputs.get("labels") if isinstance(inputs, dict) else None
        if self.compute_loss_func is not None:
            return self.compute_loss_func(outputs, labels)
        loss = outputs.get("loss") if isinstance(outputs, dict) else getattr(outputs, "loss", None)
        if loss is not None:
            return loss
        logits = outputs.get("logits") if isinstance(outputs, dict) else getattr(outputs, "logits", outputs)
        if isinstance(logits, (tuple, list)):
            logits = logits[0]
        if labels is None:
            raise ConfigurationError("the model returned no loss and the batch has no 'labels'; pass compute_loss_func")
        if logits.dim() == 3 and labels.dim() == 2:
            from ..alignment.sft.loss import nll_loss
            return nll_loss(logits, labels)[0]
        return torch.nn.functional.cross_entropy(logits.float(), labels)

    def _call_model(self, params, inputs: dict):
        """Forward pass used outside differentiation (evaluation)."""
        fmodel = self._rt.get("fmodel")
        if fmodel is None:
            return self.model(**inputs)
        return fmodel({**self._rt["frozen"], **params}, **inputs)

    # ------------------------------------------------------------------------------------------- data
    def _collate(self):
        base = self.data_collator
        if base is None:
            from torch.utils.data import default_collate
            base = default_collate
        return empty_collate(base)

    def _sampler_key(self) -> RngKey:
        seed = self.args.data_seed if self.args.data_seed is not None else self.args.seed
        return fold_in(make_key(seed), _SAMPLER_TAG)

    def get_train_dataloader(self) -> DataLoader:
        if self.train_dataset is None:
            raise ConfigurationError("training requires a train_dataset")
        rt, a = self._rt, self.args
        data = self.train_dataset
        if self.ddp.is_distributed:
            data = D.local_shard(data, rank=self.ddp.rank, world_size=self.ddp.world_size)
        base_key = self._sampler_key()
        key = fold_in(base_key, self.ddp.rank) if self.ddp.is_distributed else base_key
        sampler = mf.build_sampler(a.resolved_sampling_mode, data, sample_rate=rt["sample_rate"], n_steps=rt["total_steps"],
                                   key=key, ctx=rt.get("mf_ctx"), sampling_kwargs=a.sampling_kwargs)
        rt["sampler"], rt["sampler_stream_key"] = sampler, {"seed": base_key.seed, "impl": base_key.impl}
        kw: dict[str, Any] = {}
        if a.dataloader_num_workers > 0:
            kw.update(num_workers=a.dataloader_num_workers, persistent_workers=a.dataloader_persistent_workers,
                      prefetch_factor=a.dataloader_prefetch_factor, multiprocessing_context=a.dataloader_multiprocessing_context)
        return DataLoader(data, batch_sampler=sampler, collate_fn=self._collate(),
                          pin_memory=a.dataloader_pin_memory and self.device.type == "cuda", **kw)

    def get_eval_dataloader(self, eval_dataset=None) -> DataLoader:
        data = eval_dataset if eval_dataset is not None else self.eval_dataset
        if data is None:
            raise ConfigurationError("evaluation requires an eval_dataset")
        if self.ddp.is_distributed:
            data = D.local_shard(data, rank=self.ddp.rank, world_size=self.ddp.world_size)
        return DataLoader(data, batch_size=self.args.per_device_eval_batch_size, shuffle=False, collate_fn=self.data_collator,
                          drop_last=False, pin_memory=self.args.dataloader_pin_memory and self.device.type == "cuda")

    # ------------------------------------------------------------------------------------------- set-up
    def create_scheduler(self, total_steps: int) -> Callable[[int], float]:
        if self._user_scheduler is not None:
            self.lr_scheduler = self._user_scheduler
        else:
            a = self.args
            self.lr_scheduler = build_lr_schedule(a.lr_scheduler, learning_rate=a.learning_rate, total_steps=total_steps,
                                                  warmup_steps=a.warmup_steps or 0, kwargs=a.lr_scheduler_kwargs)
        return self.lr_scheduler

    def create_optimizer(self):
        a = self.args
        if self._user_optimizer is not None:
            self.optimizer = self._user_optimizer
        elif self._optimizer_cls_and_kwargs is not None:
            factory, kw = self._optimizer_cls_and_kwargs
            self.optimizer = factory(**kw)
        else:
            self.optimizer = build_optimizer(a.optim, lr=self.lr_scheduler, weight_decay=a.weight_decay,
                                             betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon, optim_args=a.optim_args)
        return self.optimizer

    def _resolve_clipping_norm(self, params):
        c = self.args.clipping_norm
        if isinstance(c, dict):
            kw = dict(c)
            patterns = kw.pop("patterns", None) or {k: v for k, v in kw.items() if k not in ("fallback", "allow_unused_patterns")}
            return clip_api.per_group(params, patterns, fallback=c.get("fallback"),
                                      allow_unused_patterns=bool(c.get("allow_unused_patterns", False)))
        if isinstance(c, str):
            return float(c)
        return float(c)

    def _build_process(self, nm: float):
        """Privacy process of the WHOLE run at noise multiplier ``nm``."""
        rt = self._rt
        p = rt["amplifier"](nm)
        return p * rt["total_steps"] if rt["per_step_process"] else p

    def _calibrate_noise(self) -> float:
        a, rt = self.args, self._rt
        if a.privacy_noise_multiplier is not None:
            rt["calibration_source"] = "given"
            return float(a.privacy_noise_multiplier)
        if a.privacy_target_epsilon is None:
            if a.privacy_accounting:
                raise ConfigurationError("set privacy_target_epsilon (noise is calibrated) or privacy_noise_multiplier")
            rt["calibration_source"] = "none"
            return 0.0
        kw = {"param_min": 0.05, "param_max": 200.0, **a.noise_calibration_kwargs}
        res = acc.calibrate(acc.epsilon_budget(a.privacy_target_epsilon, rt["target_delta"]), self._build_process, **kw)
        if not res.converged:
            warnings.warn(f"noise calibration stopped after {res.iterations} iterations at epsilon={res.achieved:.4f} "
                          f"(target {res.target:.4f})", stacklevel=2)
        rt["calibration_source"] = "calibrated"
        return float(res.param)

    def _setup_training(self) -> None:
        a, rt = self.args, self._rt
        n_global = len(self.train_dataset)
        if n_global == 0:
            raise ConfigurationError("train_dataset is empty")
        rt["dataset_size"] = n_global
        rt["expected_batch"] = float(a.train_batch_size)
        rt["sample_rate"] = min(1.0, a.train_batch_size / n_global)
        rt["steps_per_epoch"] = max(1, int(math.ceil(1.0 / rt["sample_rate"])))
        rt["total_steps"] = a.max_steps if a.max_steps > 0 else max(1, int(math.ceil(a.num_train_epochs * rt["steps_per_epoch"])))
        rt["target_delta"] = a.target_delta(n_global)
        self.create_scheduler(rt["total_steps"])
        # mechanism and accounting
        kind, sampling = a.privacy_noise_mechanism, a.resolved_sampling_mode
        mkw = a.resolved_mechanism_kwargs
        strategy = ctx = None
        if a.is_dpftrl:
            strategy = mf.build_strategy(kind, mkw, lr_schedule=None)
            ctx = mf.mf_context(kind, mkw, sampling, a.sampling_kwargs, n_steps=rt["total_steps"], steps_per_epoch=rt["steps_per_epoch"])
            if kind == "mf_blt" and getattr(strategy, "buf_decay", None) is None:
                # fit the buffers once so that accounting, noise generation and checkpoints see the same matrix
                strategy = strategy.optimize(ctx.n_steps, ctx.min_sep, ctx.max_participations)
        rt["strategy"], rt["mf_ctx"] = strategy, ctx
        rt["per_step_process"] = (kind == "gaussian") or (kind == "mf_identity" and sampling == "poisson")
        rt["amplifier"] = mf.build_amplifier_factory(kind, sampling, strategy=strategy, ctx=ctx, sample_rate=rt["sample_rate"],
                                                     dataset_size=n_global, n_steps=rt["total_steps"], sampling_kwargs=a.sampling_kwargs)
        rt["noise_multiplier"] = self._calibrate_noise()
        budget = acc.epsilon_budget(a.privacy_target_epsilon, rt["target_delta"]) if a.privacy_target_epsilon is not None else None
        self.accountant = acc.Accountant(budget) if a.privacy_accounting else None
        rt["step_process"] = rt["amplifier"](rt["noise_multiplier"]) if (a.privacy_accounting and rt["noise_multiplier"] > 0) else None
        self.state.noise_multiplier, self.state.sample_rate = rt["noise_multiplier"], rt["sample_rate"]
        self.state.privacy_delta = rt["target_delta"]
        if self._use_native():
            self._setup_native()
        else:
            self._setup_generic()

    def _setup_generic(self) -> None:
        a, rt = self.args, self._rt
        self.model.to(self.device)
        if a.use_performance_kernels or a.use_compat_patches:
            try:
                from .performance_kernels import apply_performance_kernels
                apply_performance_kernels(self.model, a)
            except ImportError:
                pass
        self.model.train(False)          # dropout etc. would need per-example RNG; DP fine-tuning runs deterministic forward
        if a.gradient_checkpointing or a.activation_offloading:
            # layer checkpointing that is legal under vmap(grad) (packages/opake-transformers/src/opake/api/transformers/
            # trainer/_dp_trainer.py:1499-1528): the layers re-run in the backward pass; with activation offloading the
            # kept layer inputs wait in host memory. The library checkpoints only in training mode, so dropout is zeroed.
            from ..patches.torch_checkpoint import apply_gradient_checkpointing
            from ..patches.transformers.components import disable_dropout

            disable_dropout(self.model)
            kw = {k: v for k, v in (a.gradient_checkpointing_kwargs or {}).items() if k != "use_reentrant"}
            rt["gradient_checkpointing"] = apply_gradient_checkpointing(self.model, offload=bool(a.activation_offloading), **kw)
            if rt["gradient_checkpointing"]:
                self.model.train(True)
            else:
                warnings.warn("gradient checkpointing was requested but the model exposes no checkpointing layers", stacklevel=2)
        fmodel, params, frozen = make_functional(self.model, disable_autograd_tracking=True, partition_trainable=True)
        if not params:
            raise ConfigurationError("the model has no trainable parameters")
        rt["fmodel"], rt["params"], rt["frozen"] = fmodel, params, frozen

        def call(p, **inputs):
            return fmodel({**frozen, **p}, **inputs)

        rt["loss_has_aux"] = self._overrides_metrics_seam()

        def loss_fn(p, example):
            batch = tree_map(lambda t: t.unsqueeze(0) if isinstance(t, torch.Tensor) else t, example)
            with autocast_context(a, self.device):
                if rt["loss_has_aux"]:
                    loss, tele = self.compute_per_example_loss_and_metrics(call, p, batch)
                    return loss, {k: v.detach().reshape(()) for k, v in tele.items()}
                return self.compute_per_example_loss(call, p, batch)

        norm = self._resolve_clipping_norm(params)
        common = dict(has_aux=rt["loss_has_aux"], normalize_by=rt["expected_batch"], batch_argnums=1, return_aux=True,
                      microbatch_size=self._microbatch)
        compiler = clip_api.CudaGraphChunkCompiler(max_graphs=a.cuda_graphs) if (a.cuda_graphs and self.device.type == "cuda") else None
        ckw = dict(a.clipping_kwargs)
        if a.clipping_mode == "fixed":
            grad_fn, clip_state = clip_api.clipped_grad(loss_fn, clipping_norm=norm, _chunk_compiler=compiler, **common, **ckw)
        elif a.clipping_mode == "auto":
            grad_fn, clip_state = clip_api.auto_clipped_grad(loss_fn, R=float(norm) if not hasattr(norm, "values") else 1.0,
                                                             _chunk_compiler=compiler, **common, **ckw)
        else:
            ckw.setdefault("initial_clipping_norm", float(norm) if not hasattr(norm, "values") else 1.0)
            ckw.setdefault("expected_batch_size", rt["expected_batch"])
            grad_fn, clip_state = clip_api.adaptive_clipped_grad(loss_fn, key=fold_in(make_key(a.seed), "opake.dpsgd.adaptive_clipping"),
                                                                 has_aux=rt["loss_has_aux"], normalize_by=rt["expected_batch"],
                                                                 batch_argnums=1, return_aux=True,
                                                                 microbatch_size=self._microbatch, **ckw)
            if rt["step_process"] is not None and a.privacy_noise_mechanism == "gaussian":
                from ..dpsgd import accounting as SA
                frac = float(ckw.get("fraction_noise_std", 0.05))
                base = rt["amplifier"]
                rt["amplifier"] = lambda nm, _b=base: _b(nm)      # sampling amplification applies to the joint release
                rt["step_process"] = SA.poisson(SA.adaclip(SA.gaussian(rt["noise_multiplier"]), fraction_noise_std=frac,
                                                           expected_batch_size=rt["expected_batch"]), rt["sample_rate"])
        rt["grad_fn"], rt["clip_state"] = grad_fn, clip_state
        noise_key = fold_in(make_key(a.seed), _NOISE_TAG)
        if a.is_dpftrl:
            from ..dpftrl import mf_gaussian_noise
            ctx = rt["mf_ctx"]
            rt["noise_fn"], rt["noise_state"] = mf_gaussian_noise(params, rt["strategy"], n_steps=ctx.n_steps, min_sep=ctx.min_sep,
                                                                  max_participations=ctx.max_participations,
                                                                  noise_multiplier=rt["noise_multiplier"], key=noise_key)
        else:
            rt["noise_fn"], rt["noise_state"] = sgd_noise.gaussian_noise(noise_multiplier=rt["noise_multiplier"], key=noise_key)
        self.create_optimizer()
        rt["opt_state"] = self.optimizer.init(params)

    def _setup_native(self) -> None:
        from ..parallel.engine import EngineConfig, ShardedDPEngine
        a, rt = self.args, self._rt
        norm = a.clipping_norm
        if not isinstance(norm, (int, float)):
            raise ConfigurationError("the native engine clips with one global norm; use native_engine=False for per-group clipping")
        name = a.optim.lower()
        if name not in ("adamw", "adamw-bc", "adamw_bc", "sgd", "adamw_torch", "adamw_torch_fused"):
            raise ConfigurationError(f"the native engine implements adamw, adamw-bc and sgd (got {a.optim!r})")
        blt_decay = blt_scale = ()
        nm_eff = rt["noise_multiplier"]
        if a.privacy_noise_mechanism == "mf_blt":
            ctx = rt["mf_ctx"]
            blt_decay, blt_scale = (tuple(map(float, x)) for x in rt["strategy"]._params(ctx.n_steps, ctx.min_sep, ctx.max_participations))
            # the injected noise is sigma * sens(C) * C^-1 z: the engine's buffers apply C^-1, the factor goes here
            nm_eff *= math.sqrt(rt["strategy"].sensitivity_squared(n_steps=ctx.n_steps, min_sep=ctx.min_sep,
                                                                   max_participations=ctx.max_participations))
        toeplitz_coef: tuple = ()
        if a.privacy_noise_mechanism in ("mf_band", "mf_bsr"):
            ctx = rt["mf_ctx"]
            # banded Toeplitz strategies: the engine's ring applies C^{-1} (first column = strategy coefficients), the
            # sensitivity factor of the injected noise sigma * sens(C) * C^{-1} z goes into the multiplier
            toeplitz_coef = tuple(float(x) for x in rt["strategy"].strategy_coefficients(ctx.n_steps))
            nm_eff *= math.sqrt(rt["strategy"].sensitivity_squared(n_steps=ctx.n_steps, min_sep=ctx.min_sep,
                                                                   max_participations=ctx.max_participations))
        ecfg = EngineConfig(clip_norm=float(norm), noise_multiplier=nm_eff, toeplitz_coef=toeplitz_coef, logical_batch=int(rt["expected_batch"]),
                            lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon, weight_decay=a.weight_decay,
                            noise_bias_correction=name in ("adamw-bc", "adamw_bc"), optimizer="sgd" if name == "sgd" else "adamw",
                            auto_clip=a.clipping_mode == "auto", seed=a.seed, use_cuda_graph=bool(a.cuda_graphs) or True,
                            blt_decay=tuple(blt_decay), blt_scale=tuple(blt_scale),
                            noise_stream_tag="opake.dpftrl.mf_gaussian" if a.is_dpftrl else "opake.dpsgd.gaussian")
        eng = ShardedDPEngine(self.model.cfg, ecfg, self.device, init_seed=a.seed)
        eng.params.copy_(self.model.flat.data.to(eng.params.dtype)[: eng.params.numel()] if self.model.flat.numel() >= eng.params.numel()
                         else torch.nn.functional.pad(self.model.flat.data.to(eng.params.dtype), (0, eng.params.numel() - self.model.flat.numel())))
        self._native = eng

    # ------------------------------------------------------------------------------------------- training
    def train(self, resume_from_checkpoint: str | bool | None = None, **_kw) -> TrainOutput:
        """Runs training; on a CUDA out-of-memory error in the gradient computation the micro-batch is halved and the
        run restarts from the last consistent state (all ranks step down together)."""
        resume = resume_from_checkpoint if resume_from_checkpoint is not None else self.args.resume_from_checkpoint
        while True:
            try:
                return self._train_once(resume)
            except Exception as e:  # noqa: BLE001 - classified below
                failed = _is_oom(e)
                if not failed or not self.args.auto_find_microbatch_size:
                    if self.ddp.is_distributed and failed:
                        self._cluster_needs_step_down(True)
                    raise
                self._step_down_microbatch()
                resume = resume if self.state.global_step == 0 else (ckpt.latest_checkpoint(self.args.output_dir) or resume)

    def _install_sigterm_handler(self):
        """``enable_jit_checkpoint``: SIGTERM (preemption notice) asks the loop to save a checkpoint after the step in
        flight and stop; nothing is written from inside the signal handler."""
        import signal
        self._sigterm = False
        if not self.args.enable_jit_checkpoint:
            return None
        try:
            previous = signal.getsignal(signal.SIGTERM)

            def handler(signum, frame):
                self._sigterm = True

            signal.signal(signal.SIGTERM, handler)
            return previous
        except ValueError:          # not the main thread: signals cannot be installed here
            return None

    def log_metrics(self, split: str, metrics: dict) -> None:
        if not self.ddp.is_main:
            return
        width = max((len(k) for k in metrics), default=0)
        print(f"***** {split} metrics *****")
        for k in sorted(metrics):
            v = metrics[k]
            print(f"  {k:<{width}} = {v:.6g}" if isinstance(v, float) else f"  {k:<{width}} = {v}")

    def save_metrics(self, split: str, metrics: dict, combined: bool = True) -> None:
        if not self.ddp.is_main:
            return
        os.makedirs(self.args.output_dir, exist_ok=True)
        with open(os.path.join(self.args.output_dir, f"{split}_results.json"), "w", encoding="utf-8") as f:
            json.dump(metrics, f, indent=2, sort_keys=True, default=float)
        if combined:
            path = os.path.join(self.args.output_dir, "all_results.json")
            allm = {}
            if os.path.exists(path):
                with open(path, encoding="utf-8") as f:
                    allm = json.load(f)
            allm.update(metrics)
            with open(path, "w", encoding="utf-8") as f:
                json.dump(allm, f, indent=2, sort_keys=True, default=float)

    def save_state(self) -> None:
        if self.ddp.is_main:
            os.makedirs(self.args.output_dir, exist_ok=True)
            self.state.save_to_json(os.path.join(self.args.output_dir, ckpt.FILES.TRAINER_STATE))

    def _cluster_needs_step_down(self, local: bool) -> bool:
        return bool(D.reduce_scalar(int(local), op="max")) if self.ddp.is_distributed else local

    def _step_down_microbatch(self) -> None:
        cur = self._microbatch or self.args.per_device_train_batch_size
        if cur <= 1:
            raise OperationError("out of memory even with microbatch_size=1")
        self._microbatch = max(1, cur // 2)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        warnings.warn(f"out of memory: retrying with microbatch_size={self._microbatch}", stacklevel=2)

    def _train_once(self, resume) -> TrainOutput:
        a = self.args
        self._rt = {}
        self._native = None
        self._setup_training()
        rt = self._rt
        loader = self.get_train_dataloader()
        self.callback_handler.train_dataloader = loader
        total = rt["total_steps"]
        st = self.state
        st.max_steps, st.train_batch_size = total, a.train_batch_size
        st.num_train_epochs = int(math.ceil(total / rt["steps_per_epoch"]))
        st.logging_steps = a.resolve_interval(a.logging_steps, total)
        st.save_steps = a.resolve_interval(a.save_steps, total)
        st.eval_steps = a.resolve_interval(a.eval_steps, total, fallback=a.logging_steps)
        if resume:
            path = ckpt.latest_checkpoint(a.output_dir) if resume is True else str(resume)
            if path is None or not os.path.isdir(path):
                raise CheckpointError(f"no checkpoint to resume from ({resume!r})")
            self._load_checkpoint(path)
        self.control = self.callback_handler.call_event("on_train_begin", a, st, self.control)
        previous_sigterm = self._install_sigterm_handler()
        if a.eval_on_start and self.eval_dataset is not None:
            self.evaluate()
        t0 = time.time()
        self._loss_sum, self._loss_count, self._tokens = 0.0, 0, 0
        self._tele_sum, self._tele_count = {}, 0
        run_loss, run_count = 0.0, 0
        stop_at = self._plan_stop_at_epsilon()
        if stop_at == st.global_step and st.privacy_target_epsilon_reached:        # the resumed accountant is already there
            total = st.global_step
        it = iter(loader)
        epoch_seen = -1
        while st.global_step < total:
            epoch = st.global_step // rt["steps_per_epoch"]
            if epoch != epoch_seen:
                if epoch_seen >= 0:
                    self.control = self.callback_handler.call_event("on_epoch_end", a, st, self.control)
                epoch_seen = epoch
                self.control._new_epoch()
                self.control = self.callback_handler.call_event("on_epoch_begin", a, st, self.control)
            try:
                batch = next(it)
            except StopIteration:
                break
            self.control._new_step()
            self.control = self.callback_handler.call_event("on_step_begin", a, st, self.control)
            loss, n_local = self.training_step(batch)
            st.global_step += 1
            st.epoch = st.global_step / rt["steps_per_epoch"]
            st.examples_seen += n_local
            self._loss_sum += loss
            self._loss_count += 1
            run_loss += loss
            run_count += 1
            if self.accountant is not None and rt["step_process"] is not None and rt["per_step_process"]:
                self.accountant = self.accountant | rt["step_process"]
            if stop_at is not None and st.global_step >= stop_at:
                st.privacy_target_epsilon_reached = True
                self.control.should_training_stop = True
                self.control.should_log = True
                if a.save_strategy != "no":
                    self.control.should_save = True
            self.control = self.callback_handler.call_event("on_step_end", a, st, self.control)
            self._maybe_log_save_evaluate(t0)
            if a.torch_empty_cache_steps and st.global_step % a.torch_empty_cache_steps == 0 and torch.cuda.is_available():
                torch.cuda.empty_cache()
            if self._sigterm_agreed():
                self._save_checkpoint()
                self.control.should_training_stop = True
            if self.control.should_training_stop:
                break
        if previous_sigterm is not None:
            import signal
            signal.signal(signal.SIGTERM, previous_sigterm)
        if self.accountant is not None and rt["step_process"] is not None and not rt["per_step_process"]:
            self.accountant = self.accountant | rt["step_process"]      # horizon mechanism: one process for the whole run
        if epoch_seen >= 0:
            self.control = self.callback_handler.call_event("on_epoch_end", a, st, self.control)
        self._publish_params()
        metrics = speed_metrics("train", t0, num_samples=st.examples_seen, num_steps=st.global_step,
                                num_tokens=self._tokens if a.include_tokens_per_second else None)
        metrics["train_loss"] = run_loss / max(1, run_count)
        eps = self.privacy_spent()
        if eps is not None:
            metrics["privacy_epsilon"], metrics["privacy_delta"] = eps, rt["target_delta"]
            st.privacy_epsilon = eps
        self.log(metrics)
        if a.load_best_model_at_end and st.best_model_checkpoint:
            self._load_model_weights(st.best_model_checkpoint)
        self.control = self.callback_handler.call_event("on_train_end", a, st, self.control)
        return TrainOutput(st.global_step, metrics["train_loss"], metrics)

    def _plan_stop_at_epsilon(self) -> int | None:
        """Stop-at-epsilon: with a fixed positive noise multiplier AND a target epsilon, training ends at the first step
        whose accounted epsilon reaches the target. Accounting is deterministic, so the crossing step is found once, by
        bisection over the number of steps (``predict_stop_step``); the loop then compares integers. Only defined for
        independently composed steps (not for whole-horizon mechanisms or Monte-Carlo samplers: those fall back to a
        check at every log boundary)."""
        a, rt, st = self.args, self._rt, self.state
        if not (a.privacy_noise_multiplier and a.privacy_noise_multiplier > 0 and a.privacy_target_epsilon is not None
                and self.accountant is not None and rt.get("step_process") is not None):
            return None
        if not rt["per_step_process"] or a.resolved_sampling_mode in ("b_min_sep", "balls_in_bins"):
            rt["stop_check_at_log"] = rt["per_step_process"]
            return None
        if st.global_step > 0 and self.accountant.epsilon_at(rt["target_delta"]) >= a.privacy_target_epsilon:
            st.privacy_target_epsilon_reached = True
            return st.global_step
        prefix = self.accountant.process if st.global_step > 0 else None
        stop = predict_stop_step(prefix, rt["step_process"], target_epsilon=a.privacy_target_epsilon, delta=rt["target_delta"],
                                 k0=st.global_step, horizon=rt["total_steps"])
        if stop is None:
            rt["stop_check_at_log"] = True
        return stop

    def _sigterm_agreed(self) -> bool:
        """True on every rank as soon as any rank has received SIGTERM (they must checkpoint together)."""
        if not self.args.enable_jit_checkpoint:
            return False
        flag = bool(getattr(self, "_sigterm", False))
        return bool(D.reduce_scalar(int(flag), op="max", device=self.device)) if self.ddp.is_distributed else flag

    def privacy_spent(self) -> float | None:
        """epsilon at the run's delta for everything released so far (``None`` without accounting)."""
        if self.accountant is None or not self._rt or self._rt.get("step_process") is None:
            return None
        try:
            return float(self.accountant.epsilon_at(self._rt["target_delta"]))
        except Exception:
            return None

    def training_step(self, batch) -> tuple[float, int]:
        """One DP step. Returns ``(mean example loss over the global batch, number of local examples)``."""
        if self._native is not None:
            return self._native_step(batch)
        rt, a = self._rt, self.args
        batch = _to_device(batch, self.device)
        n_local = max(0, _batch_len(batch))
        if a.include_num_input_tokens_seen and isinstance(batch, dict) and "input_ids" in batch:
            self.state.num_input_tokens_seen += int(batch["input_ids"].numel())
        with step_perf(self.device, batch_size=n_local, track_memory=not a.skip_memory_metrics) as perf:
            (grads, aux), rt["clip_state"] = rt["grad_fn"](rt["params"], batch, state=rt["clip_state"])
            perf.mark("clip")
            loss_sum = float(aux.loss_values.sum()) if getattr(aux, "loss_values", None) is not None and n_local else 0.0
            n_clipped = float(aux.clipping_rate or 0.0) * n_local if getattr(aux, "clipping_rate", None) is not None else 0.0
            tele = getattr(aux, "loss_aux", None) if rt.get("loss_has_aux") else None
            if isinstance(tele, dict) and tele:
                # per-example telemetry: local sums now, one reduction over ranks with the loss, means at the next log
                sums = {k: float(torch.as_tensor(v).float().sum()) if n_local else 0.0 for k, v in tele.items()}
                if self.ddp.is_distributed:
                    sums = {k: D.reduce_scalar(v, op="sum", device=self.device) for k, v in sorted(sums.items())}
                for k, v in sums.items():
                    self._tele_sum[k] = self._tele_sum.get(k, 0.0) + v
                self._tele_count += int(D.reduce_scalar(n_local, op="sum", device=self.device)) if self.ddp.is_distributed else n_local
            if self.ddp.is_distributed:
                D.sum_gradients_(grads)
                loss_sum = D.reduce_scalar(loss_sum, op="sum", device=self.device)
                n_clipped = D.reduce_scalar(n_clipped, op="sum", device=self.device)
                n_global = int(D.reduce_scalar(n_local, op="sum", device=self.device))
            else:
                n_global = n_local
            noised, rt["noise_state"] = rt["noise_fn"](grads, rt["noise_state"])
            perf.mark("noise")
            updates, rt["opt_state"] = self.optimizer.update(noised, rt["opt_state"], params=rt["params"])
            rt["params"] = apply_updates(rt["params"], updates)
            perf.mark("optimizer")
        self._tokens += int(batch["input_ids"].numel()) if isinstance(batch, dict) and "input_ids" in batch else 0
        self.state.clipped_fraction = n_clipped / max(1, n_global)
        return loss_sum / max(1, n_global), n_local

    def _native_step(self, batch) -> tuple[float, int]:
        eng = self._native
        ids = batch["input_ids"]
        labels = batch.get("labels", ids)
        n_local = ids.shape[0]
        # engine convention: labels already shifted (position t holds the target of t), negative = ignored
        shifted = torch.full_like(labels, -1)
        shifted[:, :-1] = torch.where(labels[:, 1:] < 0, torch.full_like(labels[:, 1:], -1), labels[:, 1:])
        tok = ids.to(torch.int32).contiguous()
        lab = shifted.to(torch.int32).contiguous()
        if self.device.type == "cuda" and not tok.is_pinned():
            tok, lab = tok.pin_memory(), lab.pin_memory()
        eng.cfg.lr = float(self.lr_scheduler(self.state.global_step))
        loss_sum = float(eng.step(tok, lab).item()) if n_local else (eng.apply_update() or 0.0)
        n_global = n_local
        if self.ddp.is_distributed:
            loss_sum = D.reduce_scalar(loss_sum, op="sum", device=self.device)
            n_global = int(D.reduce_scalar(n_local, op="sum", device=self.device))
        self._tokens += int(ids.numel())
        return loss_sum / max(1, n_global), n_local

    def _publish_params(self) -> None:
        """Copies the trained parameters back into ``self.model`` (evaluation, saving)."""
        if self._native is not None:
            with torch.no_grad():
                n = min(self.model.flat.numel(), self._native.params.numel())
                self.model.flat.data[:n].copy_(self._native.params[:n].to(self.model.flat.dtype))
            return
        params = self._rt.get("params")
        if params:
            with torch.no_grad():
                named = dict(self.model.named_parameters())
                for k, v in params.items():
                    named[k].data.copy_(v)

    def _maybe_log_save_evaluate(self, t0: float) -> None:
        a, st = self.args, self.state
        step = st.global_step
        do_log = self.control.should_log or (a.logging_strategy == "steps" and (step % st.logging_steps == 0 or (a.logging_first_step and step == 1)))
        if do_log and self._loss_count:
            logs = {"loss": self._loss_sum / self._loss_count, "learning_rate": float(self.lr_scheduler(step - 1))}
            if st.clipped_fraction is not None:
                logs["clipped_fraction"] = st.clipped_fraction
            eps = self.privacy_spent() if self._rt.get("per_step_process") else None
            if eps is not None:
                logs["privacy_epsilon"] = eps
                st.privacy_epsilon = eps
                # fallback of stop-at-epsilon when the crossing step could not be predicted (Monte-Carlo accounting)
                if self._rt.get("stop_check_at_log") and eps >= a.privacy_target_epsilon:
                    st.privacy_target_epsilon_reached = True
                    self.control.should_training_stop = True
            if getattr(self, "_tele_count", 0):
                logs.update({k: v / self._tele_count for k, v in self._tele_sum.items()})
                self._tele_sum, self._tele_count = {}, 0
            self._loss_sum, self._loss_count = 0.0, 0
            self.log(logs)
        do_eval = self.control.should_evaluate or (a.eval_strategy == "steps" and st.eval_steps and step % st.eval_steps == 0) or \
            (a.eval_strategy == "epoch" and step % self._rt["steps_per_epoch"] == 0)
        metrics = None
        if do_eval and self.eval_dataset is not None and step >= a.eval_delay:
            metrics = self.evaluate()
        do_save = self.control.should_save or (a.save_strategy == "steps" and step % st.save_steps == 0) or \
            (a.save_strategy == "epoch" and step % self._rt["steps_per_epoch"] == 0)
        if do_save:
            self._save_checkpoint(metrics)

    # ------------------------------------------------------------------------------------------- evaluation
    def prediction_step(self, inputs: dict, prediction_loss_only: bool | None = None):
        """``(per-example losses or None, logits or None, labels or None)`` for one evaluation batch (no gradients)."""
        only_loss = self.args.prediction_loss_only if prediction_loss_only is None else prediction_loss_only
        labels = inputs.get("labels") if isinstance(inputs, dict) else None
        with torch.no_grad(), autocast_context(self.args, self.device):
            params = self._rt.get("params")
            outputs = self._call_model(params, inputs) if params is not None else self.model(**inputs)
            logits = outputs.get("logits") if isinstance(outputs, dict) else getattr(outputs, "logits", None)
            losses = None
            if labels is not None or self.compute_loss_func is not None:
                if self.compute_loss_func is not None:
                    losses = self.compute_loss_func(outputs, labels)
                elif logits is not None and logits.dim() == 3 and labels.dim() == 2:
                    from ..alignment.sft.loss import nll_loss
                    losses = nll_loss(logits.float(), labels)
                elif logits is not None:
                    losses = torch.nn.functional.cross_entropy(logits.float(), labels, reduction="none")
                else:
                    loss = outputs.get("loss") if isinstance(outputs, dict) else getattr(outputs, "loss", None)
                    losses = None if loss is None else loss.reshape(1)
            if losses is not None and losses.dim() == 0:
                losses = losses.reshape(1)
        if only_loss:
            return losses, None, None
        if logits is not None and self.preprocess_logits_for_metrics is not None:
            logits = self.preprocess_logits_for_metrics(logits, labels)
        return losses, logits, labels

    def evaluation_loop(self, dataloader: DataLoader, description: str, prediction_loss_only: bool | None = None,
                        metric_key_prefix: str = "eval") -> EvaluationResult:
        a = self.args
        only_loss = (a.prediction_loss_only if prediction_loss_only is None else prediction_loss_only) or self.compute_metrics is None and description == "Evaluation"
        was_training = self.model.training
        self.model.eval()
        telemetry = EvaluationTelemetry(self.device)
        accu = PredictionAccumulator(self.device, a.eval_accumulation_steps, a.eval_do_concat_batches, telemetry=telemetry)
        n = 0
        for batch in dataloader:
            batch = _to_device(batch, self.device)
            with telemetry.model():
                losses, logits, labels = self.prediction_step(batch, only_loss)
            n += max(0, _batch_len(batch))
            accu.add(losses=losses, predictions=None if only_loss else logits, label_ids=None if only_loss else labels)
            self.control = self.callback_handler.call_event("on_prediction_step", a, self.state, self.control)
        out = accu.finalize()
        self.model.train(was_training)
        losses = out.get("losses")
        loss_sum = float(np.sum(losses)) if losses is not None else 0.0
        count = int(np.size(losses)) if losses is not None else 0
        if self.ddp.is_distributed:
            with telemetry.phase("gather"):
                loss_sum = D.reduce_scalar(loss_sum, op="sum", device=self.device)
                count = int(D.reduce_scalar(count, op="sum", device=self.device))
                n = int(D.reduce_scalar(n, op="sum", device=self.device))
        else:
            n = max(n, 0) or resolve_eval_num_samples(None, dataloader, n)
        metrics: dict[str, Any] = {}
        if count:
            metrics["loss"] = loss_sum / count
        preds, label_ids = out.get("predictions"), out.get("label_ids")
        if self.compute_metrics is not None and preds is not None:
            from types import SimpleNamespace
            with telemetry.phase("metric"):
                metrics.update(self.compute_metrics(SimpleNamespace(predictions=preds, label_ids=label_ids, losses=losses)) or {})
        tele = telemetry.to_dict()
        metrics.update(tele)        # where the evaluation time went; throughput keys are added by evaluate() / predict()
        metrics = {k: (v.item() if isinstance(v, (np.generic, torch.Tensor)) and np.size(v) == 1 else v) for k, v in metrics.items()}
        return EvaluationResult(with_metric_prefix(metrics, metric_key_prefix), n, losses, preds, label_ids, tele)

    def evaluate(self, eval_dataset=None, ignore_keys=None, metric_key_prefix: str = "eval") -> dict:
        t0 = time.time()
        if self._rt.get("params") is None and self._native is not None:
            self._publish_params()
        loader = self.get_eval_dataloader(eval_dataset)
        self.callback_handler.eval_dataloader = loader
        if self._native is not None:
            self._publish_params()
        res = self.evaluation_loop(loader, "Evaluation", metric_key_prefix=metric_key_prefix)
        metrics = {**res.metrics, **speed_metrics(metric_key_prefix, t0, num_samples=res.num_samples)}
        self.log(metrics)
        self.control = self.callback_handler.call_event("on_evaluate", self.args, self.state, self.control, metrics=metrics, trainer=self)
        self._track_best(metrics)
        return metrics

    def predict(self, test_dataset, ignore_keys=None, metric_key_prefix: str = "test") -> PredictionOutput:
        t0 = time.time()
        loader = self.get_eval_dataloader(test_dataset)
        if self._native is not None:
            self._publish_params()
        res = self.evaluation_loop(loader, "Prediction", prediction_loss_only=False, metric_key_prefix=metric_key_prefix)
        metrics = {**res.metrics, **speed_metrics(metric_key_prefix, t0, num_samples=res.num_samples)}
        self.control = self.callback_handler.call_event("on_predict", self.args, self.state, self.control, metrics=metrics)
        return PredictionOutput(res.predictions, res.label_ids, metrics)

    def _track_best(self, metrics: dict) -> None:
        name = self.args.metric_for_best_model
        if name is None:
            return
        name = name if name.startswith("eval_") else f"eval_{name}"
        if name not in metrics:
            return
        v = float(metrics[name])
        st = self.state
        if st.best_metric is None or (v > st.best_metric if self.args.greater_is_better else v < st.best_metric):
            st.best_metric, st.best_global_step = v, st.global_step
            self._best_pending = True

    # ------------------------------------------------------------------------------------------- saving
    def save_model(self, output_dir: str | None = None) -> None:
        out = output_dir or self.args.output_dir
        self._publish_params()
        if not self.ddp.is_main and not self.args.save_on_each_node:
            return
        os.makedirs(out, exist_ok=True)
        self._save_model_artifacts(out)
        if self.processing_class is not None and hasattr(self.processing_class, "save_pretrained"):
            self.processing_class.save_pretrained(out)
        torch.save(self.args.to_dict(), os.path.join(out, ckpt.FILES.TRAINING_ARGS))

    def _save_model_artifacts(self, out: str) -> None:
        m = self.model
        if hasattr(m, "save_pretrained"):
            m.save_pretrained(out, safe_serialization=self.args.save_safetensors)
            return
        sd = {k: v.detach().cpu().contiguous() for k, v in m.state_dict().items()}
        if self.args.save_safetensors:
            try:
                from safetensors.torch import save_file
                save_file(sd, os.path.join(out, ckpt.FILES.MODEL))
                return
            except Exception:       # shared tensors etc.: fall back to the pickle format
                pass
        torch.save(sd, os.path.join(out, ckpt.FILES.MODEL_PT))

    def _load_model_weights(self, path: str) -> None:
        st_path, pt_path = os.path.join(path, ckpt.FILES.MODEL), os.path.join(path, ckpt.FILES.MODEL_PT)
        if hasattr(self.model, "to_hf_state_dict") and os.path.exists(os.path.join(path, "native_config.json")):
            fresh = type(self.model).from_pretrained(path, dtype=self.model.flat.dtype, device=self.model.flat.device)
            with torch.no_grad():
                self.model.flat.data.copy_(fresh.flat.data)
        elif os.path.exists(st_path):
            from safetensors.torch import load_file
            self.model.load_state_dict(load_file(st_path), strict=False)
        elif os.path.exists(pt_path):
            self.model.load_state_dict(torch.load(pt_path, map_location="cpu", weights_only=True), strict=False)
        else:
            raise CheckpointError(f"no model weights in {path}")
        if self._rt.get("params") is not None:
            named = dict(self.model.named_parameters())
            self._rt["params"] = {k: named[k].detach().clone() for k in self._rt["params"]}
        if self._native is not None:
            n = min(self.model.flat.numel(), self._native.params.numel())
            self._native.params[:n].copy_(self.model.flat.data[:n].to(self._native.params.dtype))

    def save_accountant(self, path: str) -> None:
        if self.accountant is None:
            return
        with open(path, "w", encoding="utf-8") as f:
            json.dump(self.accountant.state_dict(), f, separators=(",", ":"), sort_keys=True)

    def _runtime_bundle(self) -> ckpt.RuntimeCheckpoint:
        rt, a = self._rt, self.args
        ctx = rt.get("mf_ctx")
        generic = self._native is None
        return ckpt.RuntimeCheckpoint(
            clip_state=state_dict(rt["clip_state"]) if generic else {}, noise_state=state_dict(rt["noise_state"]) if generic else {},
            sampler_state=rt["sampler"].state_dict(), sample_rate=rt["sample_rate"], target_delta=rt["target_delta"],
            target_epsilon=a.privacy_target_epsilon, noise_multiplier=rt["noise_multiplier"],
            expected_steps_per_epoch=rt["steps_per_epoch"], expected_batch_size=rt["expected_batch"], total_steps=rt["total_steps"],
            mechanism_kind=a.privacy_noise_mechanism, is_horizon_process=not rt["per_step_process"],
            calibration_source=rt.get("calibration_source"), mf_n_steps=ctx.n_steps if ctx else None,
            mf_min_sep=ctx.min_sep if ctx else None, mf_max_participations=ctx.max_participations if ctx else None,
            lr_scheduler=a.lr_scheduler, learning_rate=a.learning_rate, warmup_steps=a.resolve_warmup(rt["total_steps"]),
            lr_scheduler_kwargs=dict(a.lr_scheduler_kwargs), sampler_stream_key=rt.get("sampler_stream_key"))

    def _save_checkpoint(self, metrics: dict | None = None) -> str:
        a, st = self.args, self.state
        final = ckpt.checkpoint_dir(a.output_dir, st.global_step)
        stage = final + ".tmp"
        failed = False
        try:
            if self.ddp.is_main:
                shutil.rmtree(stage, ignore_errors=True)
                os.makedirs(stage, exist_ok=True)
        except OSError:
            failed = True
        checkpoint_barrier(failed, what="checkpoint staging", device=self.device)
        try:
            self._publish_params()
            if self.ddp.is_main:
                self._save_model_artifacts(stage)
                if not a.save_only_model:
                    if self._native is None:
                        torch.save(state_dict(self._rt["opt_state"]), os.path.join(stage, ckpt.FILES.OPTIMIZER))
                    ckpt.save_runtime(os.path.join(stage, ckpt.FILES.DP_STATE), self._runtime_bundle())
                    self.save_accountant(os.path.join(stage, ckpt.FILES.ACCOUNTANT))
                    st.stateful_callbacks = {type(cb).__name__: cb.state() for cb in self.callback_handler.callbacks if cb.state()}
                    st.save_to_json(os.path.join(stage, ckpt.FILES.TRAINER_STATE))
                    torch.save(a.to_dict(), os.path.join(stage, ckpt.FILES.TRAINING_ARGS))
            if not a.save_only_model:
                if self._native is not None:
                    torch.save(self._native.state_dict(), os.path.join(stage, ckpt.FILES.NATIVE_ENGINE.format(rank=self.ddp.rank)))
                ckpt.save_rng_state(os.path.join(stage, ckpt.FILES.rng(self.ddp.rank, self.ddp.world_size)))
        except Exception as e:  # noqa: BLE001 - reported to every rank through the barrier
            failed = True
            err = e
        checkpoint_barrier(failed, what="checkpoint writing", device=self.device)
        if self.ddp.is_main:
            shutil.rmtree(final, ignore_errors=True)
            os.replace(stage, final)
            if getattr(self, "_best_pending", False):
                st.best_model_checkpoint, self._best_pending = final, False
                st.save_to_json(os.path.join(final, ckpt.FILES.TRAINER_STATE))
            ckpt.rotate_checkpoints(a.output_dir, a.save_total_limit, keep=st.best_model_checkpoint)
        checkpoint_barrier(False, what="checkpoint publishing", device=self.device)
        self.control = self.callback_handler.call_event("on_save", a, st, self.control)
        return final

    def _load_checkpoint(self, path: str) -> None:
        a, rt = self.args, self._rt
        self._load_model_weights(path)
        dp_path = os.path.join(path, ckpt.FILES.DP_STATE)
        if not os.path.exists(dp_path):
            warnings.warn(f"{path} holds model weights only; optimizer, sampler and privacy state start fresh", stacklevel=2)
            return
        saved = ckpt.load_runtime(dp_path)
        ckpt.compare_runtime(saved, self._runtime_bundle())
        key_now = rt.get("sampler_stream_key")
        if saved.sampler_stream_key and key_now and saved.sampler_stream_key != key_now and not a.ignore_data_skip:
            raise CheckpointError("the sampler stream key differs from the checkpoint (seed / data_seed changed); resuming would "
                                  "re-draw examples the accountant already paid for. Set ignore_data_skip=True to start a fresh stream.")
        if a.ignore_data_skip:
            # fresh, independent sampling stream: the skipped draws are not replayed. The data loader already holds the
            # sampler object as its batch sampler, so the replacement is installed IN PLACE; under DDP the rank is folded
            # into the fresh key like it is into the original one, so ranks never share coins.
            old = rt["sampler"]
            fresh_key = fold_in(self._sampler_key(), _IGNORE_DATA_SKIP_TAG)
            if self.ddp.is_distributed:
                fresh_key = fold_in(fresh_key, self.ddp.rank)
            new = mf.build_sampler(a.resolved_sampling_mode, old.data_source if hasattr(old, "data_source") else self.train_dataset,
                                   sample_rate=rt["sample_rate"], n_steps=rt["total_steps"], ctx=rt.get("mf_ctx"),
                                   key=fresh_key, sampling_kwargs=a.sampling_kwargs)
            old.__dict__.update(new.__dict__)
        else:
            rt["sampler"].load_state_dict(_rank_local_sampler_state(saved.sampler_state, rt["sampler"], self.ddp.world_size))
        if self._native is None:
            rt["clip_state"] = from_state_dict(rt["clip_state"], saved.clip_state)
            rt["noise_state"] = from_state_dict(rt["noise_state"], saved.noise_state)
            opt_path = os.path.join(path, ckpt.FILES.OPTIMIZER)
            if os.path.exists(opt_path):
                rt["opt_state"] = from_state_dict(rt["opt_state"], torch.load(opt_path, map_location=self.device, weights_only=False))
        else:
            eng_path = os.path.join(path, ckpt.FILES.NATIVE_ENGINE.format(rank=self.ddp.rank))
            if os.path.exists(eng_path):
                self._native.load_state_dict(torch.load(eng_path, map_location="cpu", weights_only=False))
        acc_path = os.path.join(path, ckpt.FILES.ACCOUNTANT)
        if os.path.exists(acc_path) and self.accountant is not None:
            with open(acc_path, encoding="utf-8") as f:
                self.accountant = from_state_dict(self.accountant, json.load(f))
        ts_path = os.path.join(path, ckpt.FILES.TRAINER_STATE)
        if os.path.exists(ts_path):
            old = DPTrainerState.load_from_json(ts_path)
            for name in ("global_step", "epoch", "log_history", "best_metric", "best_global_step", "best_model_checkpoint",
                         "examples_seen", "num_input_tokens_seen", "privacy_epsilon"):
                setattr(self.state, name, getattr(old, name))
        ckpt.load_rng_state(os.path.join(path, ckpt.FILES.rng(self.ddp.rank, self.ddp.world_size)))

    # ------------------------------------------------------------------------------------------- hub
    def create_model_card(self, **kw) -> str:
        """Writes ``README.md`` into the output directory (process zero) and returns its text. Keywords: ``language``,
        ``license``, ``tags``, ``model_name``, ``finetuned_from`` (alias ``base_model``), ``tasks``, ``dataset_tags``,
        ``dataset``, ``dataset_args``."""
        from .hub import create_model_card

        if "base_model" in kw:
            kw.setdefault("finetuned_from", kw.pop("base_model"))
        return create_model_card(self, **kw)

    def init_hf_repo(self, token: str | None = None):
        from .hub import init_hf_repo

        return init_hf_repo(self, token=token)

    def push_to_hub(self, commit_message: str = "End of training", blocking: bool = True, token: str | None = None,
                    revision: str | None = None, **kw):
        from .hub import push_to_hub

        return push_to_hub(self, commit_message=commit_message, blocking=blocking, token=token, revision=revision, **kw)
