"""Evaluation support (packages/opake-transformers/src/opake/api/transformers/trainer/_eval.py:76-920): result
container, a prediction accumulator that keeps at most ``eval_accumulation_steps`` batches on the device and moves
the rest to pinned host memory with asynchronous copies, and the speed / prefix helpers."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

__all__ = ["EvaluationResult", "PredictionOutput", "PredictionAccumulator", "speed_metrics", "with_metric_prefix",
           "resolve_eval_num_samples"]


@dataclass
class EvaluationResult:
    metrics: dict = field(default_factory=dict)
    num_samples: int = 0
    losses: np.ndarray | None = None
    predictions: Any = None
    label_ids: Any = None


@dataclass
class PredictionOutput:
    predictions: Any
    label_ids: Any
    metrics: dict


class _HostStage:
    """Device -> pinned-host copies on a side stream; ``drain`` waits and returns numpy arrays."""

    def __init__(self, device: torch.device):
        self.device = device
        self.stream = torch.cuda.Stream(device) if device.type == "cuda" else None
        self.pending: list[tuple[torch.Tensor, Any]] = []

    def push(self, t: torch.Tensor) -> None:
        if self.stream is None:
            self.pending.append((t.detach().cpu(), None))
            return
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            host.copy_(t.detach(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        t.record_stream(self.stream)
        self.pending.append((host, ev))

    def drain(self) -> list[np.ndarray]:
        out = []
        for host, ev in self.pending:
            if ev is not None:
                ev.synchronize()
            out.append(host.float().numpy() if host.dtype == torch.bfloat16 else host.numpy())
        self.pending = []
        return out


class PredictionAccumulator:
    """Collects per-batch losses / predictions / labels. ``accumulation_steps`` bounds what stays on the device."""

    def __init__(self, device: torch.device, accumulation_steps: int | None = None, concat: bool = True):
        self.device, self.every, self.concat = device, accumulation_steps, concat
        self.fields: dict[str, _HostStage] = {}
        self.on_device: dict[str, list[torch.Tensor]] = {}
        self.batches = 0

    def add(self, **tensors: torch.Tensor | None) -> None:
        for name, t in tensors.items():
            if t is None:
                continue
            self.on_device.setdefault(name, []).append(t.detach())
        self.batches += 1
        if self.every and self.batches % self.every == 0:
            self._offload()

    def _offload(self) -> None:
        for name, items in self.on_device.items():
            stage = self.fields.setdefault(name, _HostStage(self.device))
            for t in items:
                stage.push(t)
        self.on_device = {}

    def finalize(self) -> dict[str, Any]:
        self._offload()
        out: dict[str, Any] = {}
        for name, stage in self.fields.items():
            parts = stage.drain()
            if not parts:
                continue
            if self.concat:
                try:
                    out[name] = np.concatenate([p if p.ndim else p[None] for p in parts], axis=0)
                    continue
                except ValueError:          # ragged trailing dimensions: pad to the widest
                    width = max(p.shape[1] for p in parts)
                    out[name] = np.concatenate([np.pad(p, [(0, 0), (0, width - p.shape[1])] + [(0, 0)] * (p.ndim - 2),
                                                       constant_values=-100) for p in parts], axis=0)
                    continue
            out[name] = parts
        return out


def speed_metrics(split: str, start_time: float, num_samples: int | None = None, num_steps: int | None = None,
                  num_tokens: int | None = None) -> dict:
    dt = max(time.time() - start_time, 1e-9)
    out = {f"{split}_runtime": round(dt, 4)}
    if num_samples is not None:
        out[f"{split}_samples_per_second"] = round(num_samples / dt, 3)
    if num_steps is not None:
        out[f"{split}_steps_per_second"] = round(num_steps / dt, 3)
    if num_tokens is not None:
        out[f"{split}_tokens_per_second"] = round(num_tokens / dt, 3)
    return out


def with_metric_prefix(metrics: dict, prefix: str) -> dict:
    return {(k if k.startswith(f"{prefix}_") else f"{prefix}_{k}"): v for k, v in metrics.items()}


def resolve_eval_num_samples(dataset, dataloader, observed: int) -> int:
    try:
        return len(dataset)
    except TypeError:
        return observed
