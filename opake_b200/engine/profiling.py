"""Step timing and memory accounting.

Same objects as packages/opake-engine/src/opake/api/engine/profiling/_memory.py:51-744 (``MemoryStats``, ``StepPerf``,
``step_perf`` with ``.mark(name)``, ``PerfState``, ``PerfStage``, ``PerfTracker``) with one B200-specific change:
on CUDA the marks are CUDA events recorded on the current stream and resolved once at the end of the step, so timing
a step does not insert a device synchronisation per mark. Cross-rank aggregation (:func:`sync_perf_state`) takes
time = max over ranks, samples = sum, peak memory = max.
"""
from __future__ import annotations

import time
from collections.abc import Mapping
from contextlib import contextmanager
from dataclasses import dataclass, field, replace
from types import MappingProxyType

import torch

_GB = 1024**3


@dataclass(frozen=True)
class MemoryStats:
    allocated_gb: float = 0.0
    reserved_gb: float = 0.0
    peak_gb: float = 0.0
    free_gb: float = 0.0
    total_gb: float = 0.0
    exact_peak: bool = False
    exact_reserved: bool = False
    known_free: bool = False
    known_total: bool = False

    @property
    def utilization(self) -> float:
        return self.allocated_gb / self.total_gb if self.total_gb > 0 else 0.0

    def to_dict(self, prefix: str = "memory/") -> dict:
        return {f"{prefix}allocated_gb": self.allocated_gb, f"{prefix}reserved_gb": self.reserved_gb,
                f"{prefix}peak_gb": self.peak_gb, f"{prefix}free_gb": self.free_gb, f"{prefix}total_gb": self.total_gb,
                f"{prefix}utilization": self.utilization}

    def __str__(self) -> str:
        return (f"allocated {self.allocated_gb:.2f} GB, reserved {self.reserved_gb:.2f} GB, peak {self.peak_gb:.2f} GB, "
                f"free {self.free_gb:.2f}/{self.total_gb:.2f} GB")


def get_memory_stats(device) -> MemoryStats:
    dev = torch.device(device)
    if dev.type == "cuda" and torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info(dev)
        return MemoryStats(torch.cuda.memory_allocated(dev) / _GB, torch.cuda.memory_reserved(dev) / _GB,
                           torch.cuda.max_memory_allocated(dev) / _GB, free / _GB, total / _GB, True, True, True, True)
    try:
        import psutil

        vm = psutil.virtual_memory()
        rss = psutil.Process().memory_info().rss
        return MemoryStats(rss / _GB, rss / _GB, rss / _GB, vm.available / _GB, vm.total / _GB, known_free=True,
                           known_total=True)
    except Exception:
        return MemoryStats()


def reset_peak_memory(device) -> None:
    dev = torch.device(device)
    if dev.type == "cuda" and torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats(dev)


def print_memory(device, label: str = "") -> MemoryStats:
    st = get_memory_stats(device)
    print(f"[memory{' ' + label if label else ''}] {st}")
    return st


def empty_cache(device) -> None:
    if torch.device(device).type == "cuda" and torch.cuda.is_available():
        torch.cuda.empty_cache()


@dataclass(frozen=True)
class StepPerf:
    step_time_sec: float = 0.0
    samples_per_second: float = 0.0
    memory_peak_gb: float = 0.0
    memory_allocated_gb: float = 0.0
    memory_reserved_gb: float = 0.0
    batch_size: int = 0
    marks: Mapping[str, float] = field(default_factory=lambda: MappingProxyType({}))

    def to_dict(self, prefix: str = "") -> dict[str, float]:
        d = {f"{prefix}step_time_sec": self.step_time_sec, f"{prefix}samples_per_second": self.samples_per_second,
             f"{prefix}memory_peak_gb": self.memory_peak_gb, f"{prefix}batch_size": float(self.batch_size)}
        for k, v in self.marks.items():
            d[f"{prefix}time/{k}"] = v
        return d


class _StepPerfBuilder:
    def __init__(self, device: torch.device, batch_size: int, track_memory: bool):
        self.device, self.batch_size, self.track_memory = device, batch_size, track_memory
        self.cuda = device.type == "cuda" and torch.cuda.is_available()
        self._names: list[str] = []
        self._events = []
        self._times = []
        self._result: StepPerf | None = None
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record(torch.cuda.current_stream(device))
            self._events.append(e)
        else:
            self._times.append(time.perf_counter())

    def mark(self, name: str) -> None:
        """End of phase ``name`` (device-timed on CUDA, wall-clock on CPU)."""
        self._names.append(name)
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record(torch.cuda.current_stream(self.device))
            self._events.append(e)
        else:
            self._times.append(time.perf_counter())

    def finish(self) -> StepPerf:
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record(torch.cuda.current_stream(self.device))
            e.synchronize()
            stamps = [0.0] + [self._events[0].elapsed_time(x) / 1e3 for x in self._events[1:]]
            total = self._events[0].elapsed_time(e) / 1e3
        else:
            now = time.perf_counter()
            stamps = [t - self._times[0] for t in self._times]
            total = now - self._times[0]
        marks = {n: stamps[i + 1] - stamps[i] for i, n in enumerate(self._names)}
        mem = get_memory_stats(self.device) if self.track_memory else MemoryStats()
        self._result = StepPerf(total, self.batch_size / total if total > 0 else 0.0, mem.peak_gb, mem.allocated_gb,
                                mem.reserved_gb, self.batch_size, MappingProxyType(marks))
        return self._result

    @property
    def perf(self) -> StepPerf:
        return self._result if self._result is not None else self.finish()

    result = perf


@contextmanager
def step_perf(device, *, batch_size: int = 0, track_memory: bool = True):
    b = _StepPerfBuilder(torch.device(device), batch_size, track_memory)
    try:
        yield b
    finally:
        b.finish()


@dataclass(frozen=True)
class PerfState:
    device: torch.device
    num_steps: int = 0
    total_time: float = 0.0
    total_samples: int = 0
    num_steps_stable: int = 0
    total_time_stable: float = 0.0
    total_samples_stable: int = 0
    max_peak_memory_gb: float = 0.0
    last_step: StepPerf | None = None
    warmup_steps: int = 1

    def add(self, perf: StepPerf) -> "PerfState":
        stable = self.num_steps >= self.warmup_steps
        return replace(self, num_steps=self.num_steps + 1, total_time=self.total_time + perf.step_time_sec,
                       total_samples=self.total_samples + perf.batch_size,
                       num_steps_stable=self.num_steps_stable + (1 if stable else 0),
                       total_time_stable=self.total_time_stable + (perf.step_time_sec if stable else 0.0),
                       total_samples_stable=self.total_samples_stable + (perf.batch_size if stable else 0),
                       max_peak_memory_gb=max(self.max_peak_memory_gb, perf.memory_peak_gb), last_step=perf)

    @property
    def avg_step_time(self) -> float:
        return self.total_time / self.num_steps if self.num_steps else 0.0

    @property
    def avg_step_time_stable(self) -> float:
        return self.total_time_stable / self.num_steps_stable if self.num_steps_stable else self.avg_step_time

    @property
    def avg_samples_per_second(self) -> float:
        return self.total_samples / self.total_time if self.total_time > 0 else 0.0

    @property
    def avg_samples_per_second_stable(self) -> float:
        return self.total_samples_stable / self.total_time_stable if self.total_time_stable > 0 else self.avg_samples_per_second

    def to_dict(self, prefix: str = "") -> dict[str, float]:
        return {f"{prefix}num_steps": float(self.num_steps), f"{prefix}avg_step_time": self.avg_step_time_stable,
                f"{prefix}samples_per_second": self.avg_samples_per_second_stable,
                f"{prefix}max_peak_memory_gb": self.max_peak_memory_gb}


class PerfStage:
    """Mutable accumulator for one stage (train / eval / test); ``stage |= perf`` or ``with stage(batch_size=n):``."""

    def __init__(self, device: torch.device, warmup_steps: int = 1, name: str = ""):
        self.name = name
        self.state = PerfState(device=device, warmup_steps=warmup_steps)

    @property
    def samples_per_second(self) -> float:
        return self.state.avg_samples_per_second_stable

    @property
    def steps_per_second(self) -> float:
        t = self.state.avg_step_time_stable
        return 1.0 / t if t > 0 else 0.0

    def __ior__(self, perf: StepPerf) -> "PerfStage":
        self.state = self.state.add(perf)
        return self

    @contextmanager
    def __call__(self, *, batch_size: int = 0, track_memory: bool = True):
        with step_perf(self.state.device, batch_size=batch_size, track_memory=track_memory) as b:
            yield b
        self.state = self.state.add(b.perf)

    def to_dict(self, prefix: str = "") -> dict[str, float]:
        return self.state.to_dict(prefix or (self.name + "/" if self.name else ""))


class PerfTracker:
    """``tracker.train`` / ``tracker.eval`` / ``tracker["anything"]`` create stages on first use."""

    def __init__(self, device: torch.device, warmup_steps: int = 1):
        object.__setattr__(self, "_device", device)
        object.__setattr__(self, "_warmup", warmup_steps)
        object.__setattr__(self, "_stages", {})

    def _get(self, name: str) -> PerfStage:
        st = self._stages.get(name)
        if st is None:
            st = self._stages[name] = PerfStage(self._device, self._warmup, name)
        return st

    def __getattr__(self, name: str) -> PerfStage:
        if name.startswith("_"):
            raise AttributeError(name)
        return self._get(name)

    def __setattr__(self, name: str, value) -> None:
        if isinstance(value, PerfStage):
            self._stages[name] = value
        else:
            object.__setattr__(self, name, value)

    def __getitem__(self, name: str) -> PerfStage:
        return self._get(name)

    def stages(self) -> dict[str, PerfStage]:
        return dict(self._stages)


def perf_tracker(device, warmup_steps: int = 1) -> PerfTracker:
    return PerfTracker(torch.device(device), warmup_steps)


def sync_perf_state(state: PerfState) -> PerfState:
    """Cross-rank view: times are the max over ranks, samples the sum, peak memory the max."""
    from . import distributed as D

    if not D.is_distributed():
        return state
    dev = state.device if state.device.type == "cuda" else None
    return replace(state, total_time=D.reduce_scalar(state.total_time, "max", dev),
                   total_time_stable=D.reduce_scalar(state.total_time_stable, "max", dev),
                   total_samples=D.reduce_scalar(state.total_samples, "sum", dev),
                   total_samples_stable=D.reduce_scalar(state.total_samples_stable, "sum", dev),
                   max_peak_memory_gb=D.reduce_scalar(state.max_peak_memory_gb, "max", dev))


__all__ = ["nvtx_range", "PerfStage", "PerfState", "PerfTracker", "StepPerf", "MemoryStats", "empty_cache", "get_memory_stats",
           "perf_tracker", "print_memory", "reset_peak_memory", "step_perf", "sync_perf_state"]


class nvtx_range:
    """NVTX range around a phase (shows up in Nsight Systems / Compute timelines); a no-op without CUDA. Also opens a
    ``torch.profiler.record_function`` range of the same name, so the phase is visible to both kinds of tools."""

    def __init__(self, name: str):
        self.name = name
        self._rf = None
        self._pushed = False

    def __enter__(self):
        import torch

        if torch.cuda.is_available():
            try:
                torch.cuda.nvtx.range_push(self.name)
                self._pushed = True
            except Exception:       # NVTX not built into this torch
                self._pushed = False
        self._rf = torch.profiler.record_function(self.name)
        self._rf.__enter__()
        return self

    def __exit__(self, *exc):
        import torch

        self._rf.__exit__(*exc)
        if self._pushed:
            torch.cuda.nvtx.range_pop()
        return False
