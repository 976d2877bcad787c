"""Callback protocol of the trainer (packages/opake-transformers/src/opake/api/transformers/trainer/
_callback.py:190-353): the Hugging Face event names, a handler that fans events out, console / TensorBoard /
Weights & Biases reporters (imported lazily, skipped when the package is missing) and best-model saving."""
from __future__ import annotations

import json
import os
from typing import Any

from .state import DPTrainerState, TrainerControl

__all__ = ["TrainerCallback", "CallbackHandler", "PrinterCallback", "TensorBoardCallback", "WandbCallback",
           "BestModelSaveCallback", "EarlyStoppingCallback", "JsonlLoggerCallback", "reporting_callbacks"]

_EVENTS = ("on_init_end", "on_train_begin", "on_train_end", "on_epoch_begin", "on_epoch_end", "on_step_begin",
           "on_step_end", "on_evaluate", "on_predict", "on_save", "on_log", "on_prediction_step", "on_push_begin")


class TrainerCallback:
    """Subclass and override any event; each receives ``(args, state, control, **kwargs)`` and may return a control."""

    def on_init_end(self, args, state, control, **kw): ...
    def on_train_begin(self, args, state, control, **kw): ...
    def on_train_end(self, args, state, control, **kw): ...
    def on_epoch_begin(self, args, state, control, **kw): ...
    def on_epoch_end(self, args, state, control, **kw): ...
    def on_step_begin(self, args, state, control, **kw): ...
    def on_step_end(self, args, state, control, **kw): ...
    def on_evaluate(self, args, state, control, **kw): ...
    def on_predict(self, args, state, control, **kw): ...
    def on_save(self, args, state, control, **kw): ...
    def on_log(self, args, state, control, **kw): ...
    def on_prediction_step(self, args, state, control, **kw): ...
    def on_push_begin(self, args, state, control, **kw): ...

    def state(self) -> dict:            # stateful callbacks may persist themselves in trainer_state.json
        return {}


class CallbackHandler:
    def __init__(self, callbacks, model=None, processing_class=None, optimizer=None, lr_scheduler=None):
        self.callbacks: list[TrainerCallback] = []
        for cb in callbacks or []:
            self.add_callback(cb)
        self.model, self.processing_class, self.optimizer, self.lr_scheduler = model, processing_class, optimizer, lr_scheduler
        self.train_dataloader = self.eval_dataloader = None

    def add_callback(self, cb):
        cb = cb() if isinstance(cb, type) else cb
        self.callbacks.append(cb)

    def pop_callback(self, cb):
        for c in self.callbacks:
            if c is cb or (isinstance(cb, type) and isinstance(c, cb)):
                self.callbacks.remove(c)
                return c
        return None

    def remove_callback(self, cb):
        self.pop_callback(cb)

    def call_event(self, event: str, args, state: DPTrainerState, control: TrainerControl, **kw) -> TrainerControl:
        assert event in _EVENTS, event
        for cb in self.callbacks:
            out = getattr(cb, event)(args, state, control, model=self.model, processing_class=self.processing_class,
                                     optimizer=self.optimizer, lr_scheduler=self.lr_scheduler,
                                     train_dataloader=self.train_dataloader, eval_dataloader=self.eval_dataloader, **kw)
            if out is not None:
                control = out
        return control


class PrinterCallback(TrainerCallback):
    def on_log(self, args, state, control, logs=None, **kw):
        if state.is_world_process_zero and logs:
            print({k: (round(v, 6) if isinstance(v, float) else v) for k, v in logs.items()}, flush=True)


class JsonlLoggerCallback(TrainerCallback):
    """Appends every log record to ``<logging_dir or output_dir>/metrics.jsonl``."""

    def on_log(self, args, state, control, logs=None, **kw):
        if not state.is_world_process_zero or not logs:
            return
        root = args.logging_dir or args.output_dir
        os.makedirs(root, exist_ok=True)
        with open(os.path.join(root, "metrics.jsonl"), "a", encoding="utf-8") as f:
            f.write(json.dumps({"step": state.global_step, **logs}, default=float) + "\n")


class TensorBoardCallback(TrainerCallback):
    def __init__(self):
        self.writer = None

    def on_train_begin(self, args, state, control, **kw):
        if not state.is_world_process_zero:
            return
        try:
            from torch.utils.tensorboard import SummaryWriter
        except Exception:                       # tensorboard not installed: reporting silently off
            return
        self.writer = SummaryWriter(log_dir=args.logging_dir or os.path.join(args.output_dir, "runs"))

    def on_log(self, args, state, control, logs=None, **kw):
        if self.writer is None or not logs:
            return
        for k, v in logs.items():
            if isinstance(v, (int, float)):
                self.writer.add_scalar(k, v, state.global_step)
        self.writer.flush()

    def on_train_end(self, args, state, control, **kw):
        if self.writer is not None:
            self.writer.close()
            self.writer = None


class WandbCallback(TrainerCallback):
    def __init__(self):
        self.run = None

    def on_train_begin(self, args, state, control, **kw):
        if not state.is_world_process_zero:
            return
        try:
            import wandb
        except Exception:
            return
        self.run = wandb.init(project=args.project or "opake", name=args.run_name, config=args.to_dict())

    def on_log(self, args, state, control, logs=None, **kw):
        if self.run is not None and logs:
            self.run.log({k: v for k, v in logs.items() if isinstance(v, (int, float))}, step=state.global_step)

    def on_train_end(self, args, state, control, **kw):
        if self.run is not None:
            self.run.finish()
            self.run = None


class BestModelSaveCallback(TrainerCallback):
    """Saves the model to ``<output_dir>/best`` whenever the tracked evaluation metric improves."""

    def __init__(self, metric: str = "eval_loss", greater_is_better: bool = False, subdir: str = "best"):
        self.metric, self.greater, self.subdir, self.best = metric, greater_is_better, subdir, None

    def on_evaluate(self, args, state, control, metrics=None, trainer=None, **kw):
        if not metrics or self.metric not in metrics:
            return
        v = float(metrics[self.metric])
        if self.best is None or (v > self.best if self.greater else v < self.best):
            self.best = v
            if trainer is not None:
                trainer.save_model(os.path.join(args.output_dir, self.subdir))

    def state(self) -> dict:
        return {"best": self.best}


class EarlyStoppingCallback(TrainerCallback):
    def __init__(self, early_stopping_patience: int = 1, early_stopping_threshold: float = 0.0):
        self.patience, self.threshold, self.bad, self.best = early_stopping_patience, early_stopping_threshold, 0, None

    def on_evaluate(self, args, state, control, metrics=None, **kw):
        name = args.metric_for_best_model or "loss"
        name = name if name.startswith("eval_") else f"eval_{name}"
        if not metrics or name not in metrics:
            return
        v = float(metrics[name])
        better = self.best is None or ((v > self.best + self.threshold) if args.greater_is_better else (v < self.best - self.threshold))
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                control.should_training_stop = True
        return control


def reporting_callbacks(report_to) -> list[TrainerCallback]:
    out: list[TrainerCallback] = []
    for name in report_to or []:
        if name == "tensorboard":
            out.append(TensorBoardCallback())
        elif name == "wandb":
            out.append(WandbCallback())
        elif name in ("jsonl", "json"):
            out.append(JsonlLoggerCallback())
    return out
