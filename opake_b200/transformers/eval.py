"""Evaluation support (packages/opake-transformers/src/opake/api/transformers/trainer/_eval.py:76-920).

* :class:`EvaluationTelemetry`: where evaluation time goes (model, gather, device-to-host transfer, finalisation,
  metric function) without serialising the GPU: model and transfer intervals are CUDA events resolved once at the
  end, and the part of the transfer time hidden under model work is reported as ``transfer_overlap_sec``.
* :class:`TransferPipeline`: device -> pinned-host copies on a side stream with at most ``max_pending`` payloads in
  flight (bounds pinned memory), nested payloads (tensors inside tuples / lists / dicts) kept in shape.
* :class:`PredictionAccumulator`: per-batch losses / predictions / labels; at most ``eval_accumulation_steps`` batches
  stay on the device, the rest are moved to the host while the next batches run; ragged trailing dimensions are
  padded with -100 (the ignore value metric functions mask) when batches are concatenated.
* ``speed_metrics``, ``with_metric_prefix``, ``resolve_eval_num_samples``.
"""
from __future__ import annotations

import time
from collections import deque
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, Mapping

import numpy as np
import torch

__all__ = ["EvaluationResult", "PredictionOutput", "PredictionAccumulator", "EvaluationTelemetry", "TransferPipeline",
           "speed_metrics", "with_metric_prefix", "resolve_eval_num_samples", "PAD_VALUE"]

PAD_VALUE = -100


@dataclass
class EvaluationResult:
    metrics: dict = field(default_factory=dict)
    num_samples: int = 0
    losses: np.ndarray | None = None
    predictions: Any = None
    label_ids: Any = None
    telemetry: dict = field(default_factory=dict)


@dataclass
class PredictionOutput:
    predictions: Any
    label_ids: Any
    metrics: dict


# --------------------------------------------------------------------------------------------------- telemetry
def interval_overlap(left: list[tuple[float, float]], right: list[tuple[float, float]]) -> float:
    """Total overlap of two chronologically ordered interval lists (two-pointer sweep)."""
    total, i, j = 0.0, 0, 0
    while i < len(left) and j < len(right):
        (a0, a1), (b0, b1) = left[i], right[j]
        total += max(0.0, min(a1, b1) - max(a0, b0))
        if a1 <= b1:
            i += 1
        else:
            j += 1
    return total


@dataclass
class EvaluationTelemetry:
    device: torch.device
    model_time_sec: float = 0.0
    gather_time_sec: float = 0.0
    transfer_time_sec: float = 0.0
    finalization_time_sec: float = 0.0
    metric_time_sec: float = 0.0
    transfer_bytes: int = 0
    transfer_overlap_sec: float = 0.0
    _origin: Any = field(default=None, init=False, repr=False)
    _model_events: list = field(default_factory=list, init=False, repr=False)
    _transfer_events: list = field(default_factory=list, init=False, repr=False)
    _finished: bool = field(default=False, init=False, repr=False)

    def __post_init__(self):
        self.device = torch.device(self.device)
        if self.device.type == "cuda":
            self._origin = torch.cuda.Event(enable_timing=True)
            self._origin.record(torch.cuda.current_stream(self.device))

    @contextmanager
    def model(self):
        if self.device.type == "cuda":
            stream = torch.cuda.current_stream(self.device)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            yield
            b.record(stream)
            self._model_events.append((a, b))
            return
        t0 = time.perf_counter()
        yield
        self.model_time_sec += time.perf_counter() - t0

    @contextmanager
    def phase(self, name: str):
        """Host-timed phase: ``gather``, ``transfer``, ``finalization`` or ``metric``."""
        t0 = time.perf_counter()
        yield
        key = f"{name}_time_sec"
        setattr(self, key, getattr(self, key) + time.perf_counter() - t0)

    def add_transfer(self, *, num_bytes: int, events: tuple | None = None, elapsed_sec: float = 0.0) -> None:
        self.transfer_bytes += int(num_bytes)
        self.transfer_time_sec += elapsed_sec
        if events is not None:
            self._transfer_events.append(events)

    def finish(self) -> None:
        if self._finished:
            return
        self._finished = True
        if self.device.type != "cuda":
            return
        torch.cuda.synchronize(self.device)
        self.model_time_sec += sum(a.elapsed_time(b) for a, b in self._model_events) / 1e3
        self.transfer_time_sec += sum(a.elapsed_time(b) for a, b in self._transfer_events) / 1e3
        rel = lambda evs: [(self._origin.elapsed_time(a) / 1e3, self._origin.elapsed_time(b) / 1e3) for a, b in evs]  # noqa: E731
        self.transfer_overlap_sec = interval_overlap(rel(self._model_events), rel(self._transfer_events))

    def to_dict(self) -> dict:
        self.finish()
        ratio = self.transfer_overlap_sec / self.transfer_time_sec if self.transfer_time_sec > 0 else 0.0
        return {"model_time_sec": self.model_time_sec, "gather_time_sec": self.gather_time_sec,
                "transfer_time_sec": self.transfer_time_sec, "finalization_time_sec": self.finalization_time_sec,
                "metric_time_sec": self.metric_time_sec, "transfer_bytes": self.transfer_bytes,
                "transfer_overlap_sec": self.transfer_overlap_sec, "transfer_overlap_ratio": ratio}


# --------------------------------------------------------------------------------------------------- nested payloads
def _map_nested(fn, value):
    if isinstance(value, torch.Tensor):
        return fn(value)
    if isinstance(value, Mapping):
        return type(value)((k, _map_nested(fn, v)) for k, v in value.items())
    if isinstance(value, tuple) and hasattr(value, "_fields"):
        return type(value)(*(_map_nested(fn, v) for v in value))
    if isinstance(value, (list, tuple)):
        return type(value)(_map_nested(fn, v) for v in value)
    return value


def _tensors(value) -> list[torch.Tensor]:
    out: list[torch.Tensor] = []
    _map_nested(lambda t: out.append(t) or t, value)
    return out


def nested_num_bytes(value) -> int:
    return sum(t.numel() * t.element_size() for t in _tensors(value))


def _to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach()
    return (t.float() if t.dtype in (torch.bfloat16, torch.float16) else t).cpu().numpy()


class TransferPipeline:
    """At most ``max_pending`` staged payloads wait for their copies; submitting one more first drains the oldest."""

    def __init__(self, telemetry: EvaluationTelemetry | None = None, max_pending: int = 2):
        self.telemetry, self.max_pending = telemetry, max(1, int(max_pending))
        self._pending: deque = deque()
        self._stream = None
        self.max_pending_observed = 0

    def submit(self, payload) -> list:
        """Starts the copy of ``payload``; returns the payloads whose copies completed (host, numpy leaves)."""
        cuda = [t for t in _tensors(payload) if t.is_cuda]
        if not cuda:
            t0 = time.perf_counter()
            host = _map_nested(_to_numpy, payload)
            if self.telemetry is not None:
                self.telemetry.add_transfer(num_bytes=nested_num_bytes(payload), elapsed_sec=time.perf_counter() - t0)
            return [host]
        done = []
        if len(self._pending) >= self.max_pending:
            done.append(self._drain_one())
        device = cuda[0].device
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=device)
        self._stream.wait_stream(torch.cuda.current_stream(device))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def stage(t: torch.Tensor) -> torch.Tensor:
            if not t.is_cuda:
                return t.detach()
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            host.copy_(t.detach(), non_blocking=True)
            t.record_stream(self._stream)
            return host

        with torch.cuda.stream(self._stream):
            a.record(self._stream)
            staged = _map_nested(stage, payload)
            b.record(self._stream)
        self._pending.append((staged, a, b, nested_num_bytes(payload)))
        self.max_pending_observed = max(self.max_pending_observed, len(self._pending))
        return done

    def _drain_one(self):
        staged, a, b, nbytes = self._pending.popleft()
        b.synchronize()
        if self.telemetry is not None:
            self.telemetry.add_transfer(num_bytes=nbytes, events=(a, b))
        return _map_nested(_to_numpy, staged)        # numpy copies: the pinned staging buffers are released

    def drain_all(self) -> list:
        return [self._drain_one() for _ in range(len(self._pending))]


# --------------------------------------------------------------------------------------------------- accumulator
def _concat_arrays(parts: list[np.ndarray]) -> np.ndarray:
    parts = [p if p.ndim else p[None] for p in parts]
    try:
        return np.concatenate(parts, axis=0)
    except ValueError:      # ragged trailing dimensions: pad every axis but the first to the widest, with -100
        nd = max(p.ndim for p in parts)
        if any(p.ndim != nd for p in parts):
            raise
        widest = [max(p.shape[ax] for p in parts) for ax in range(1, nd)]
        padded = [np.pad(p, [(0, 0)] + [(0, w - s) for w, s in zip(widest, p.shape[1:])], constant_values=PAD_VALUE)
                  for p in parts]
        return np.concatenate(padded, axis=0)


def concat_nested(parts: list):
    """Concatenates a list of equally structured payloads leaf by leaf along the batch axis."""
    first = parts[0]
    if isinstance(first, np.ndarray):
        return _concat_arrays(parts)
    if isinstance(first, Mapping):
        return type(first)((k, concat_nested([p[k] for p in parts])) for k in first)
    if isinstance(first, (list, tuple)):
        return type(first)(concat_nested([p[i] for p in parts]) for i in range(len(first)))
    return first


class PredictionAccumulator:
    """Collects per-batch losses / predictions / labels. ``accumulation_steps`` bounds what stays on the device; values
    may be tensors or nested containers of tensors (models that return several prediction heads)."""

    def __init__(self, device: torch.device, accumulation_steps: int | None = None, concat: bool = True,
                 telemetry: EvaluationTelemetry | None = None, max_pending_transfers: int = 2):
        self.device, self.every, self.concat = torch.device(device), accumulation_steps, concat
        self.telemetry = telemetry
        self.pipeline = TransferPipeline(telemetry, max_pending_transfers)
        self.on_device: list[dict] = []
        self.host: list[dict] = []
        self.batches = 0

    def add(self, **values) -> None:
        entry = {k: _map_nested(lambda t: t.detach(), v) for k, v in values.items() if v is not None}
        self.on_device.append(entry)
        self.batches += 1
        if self.every and self.batches % self.every == 0:
            self.flush_to_cpu()

    def flush_to_cpu(self) -> None:
        """Starts moving everything held on the device to the host; completed copies are collected as they finish."""
        if not self.on_device:
            return
        with (self.telemetry.phase("gather") if self.telemetry is not None else _null()):
            chunk, self.on_device = self.on_device, []
        self.host.extend(self.pipeline.submit(chunk))

    def finalize(self) -> dict[str, Any]:
        self.flush_to_cpu()
        self.host.extend(self.pipeline.drain_all())
        with (self.telemetry.phase("finalization") if self.telemetry is not None else _null()):
            entries = [e for chunk in self.host for e in chunk]          # chunks are lists of per-batch dicts, in order
            out: dict[str, Any] = {}
            for name in {k for e in entries for k in e}:
                parts = [e[name] for e in entries if name in e]
                out[name] = concat_nested(parts) if self.concat else parts
            self.host = []
        return out


@contextmanager
def _null():
    yield


# --------------------------------------------------------------------------------------------------- helpers
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


def resolve_eval_num_samples(dataset, dataloader=None, observed: int = 0) -> int:
    """Size of the evaluation set: the dataset's length when it has one (a sharded or dropping loader observes fewer),
    else the loader's dataset, else the number of examples actually seen."""
    for obj in (dataset, getattr(dataloader, "dataset", None)):
        try:
            if obj is not None:
                return len(obj)
        except TypeError:
            continue
    return int(observed)
