"""Checkpoint files of the trainer (packages/opake-transformers/src/opake/api/transformers/trainer/
_checkpoint.py:34-415). A checkpoint is a directory ``checkpoint-<step>`` staged as ``checkpoint-<step>.tmp`` and
renamed when complete. ``dp_state.pt`` holds a ``RuntimeCheckpoint`` (bundle version 8): flat state dicts of the
clipping, noise and sampler states plus the scalars that must match on resume. Each scalar has a drift class:
``dp_relevant`` values change the privacy analysis (DP-SGD warns, horizon / DP-FTRL runs refuse to resume),
``intentional_extend`` may grow (training longer with Gaussian noise just spends more), ``shape`` values only change
the learning-rate curve."""
from __future__ import annotations

import dataclasses
import os
import random
import re
import shutil
import warnings
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from ..base.exceptions import CheckpointError

__all__ = ["RuntimeCheckpoint", "BUNDLE_VERSION", "FILES", "checkpoint_dir", "list_checkpoints", "latest_checkpoint",
           "rotate_checkpoints", "save_runtime", "load_runtime", "save_rng_state", "load_rng_state", "compare_runtime"]

BUNDLE_VERSION = 8
PREFIX = "checkpoint"


class FILES:
    TRAINER_STATE = "trainer_state.json"
    TRAINING_ARGS = "training_args.bin"
    OPTIMIZER = "dp_optimizer.pt"
    DP_STATE = "dp_state.pt"
    ACCOUNTANT = "accountant.json"
    RNG = "rng_state.pth"
    MODEL = "model.safetensors"
    MODEL_PT = "pytorch_model.bin"
    NATIVE_ENGINE = "native_engine_rank{rank}.pt"

    @staticmethod
    def rng(rank: int, world: int) -> str:
        return "rng_state.pth" if world <= 1 else f"rng_state_{rank}.pth"


DP_RELEVANT = ("sample_rate", "target_delta", "noise_multiplier", "expected_steps_per_epoch", "expected_batch_size",
               "mechanism_kind", "is_horizon_process", "mf_n_steps", "mf_min_sep", "mf_max_participations",
               "sampler_stream_key")
SHAPE = ("lr_scheduler", "learning_rate", "warmup_steps", "lr_scheduler_kwargs")


@dataclass
class RuntimeCheckpoint:
    version: int = BUNDLE_VERSION
    clip_state: dict = field(default_factory=dict)
    noise_state: dict = field(default_factory=dict)
    sampler_state: dict = field(default_factory=dict)
    sample_rate: float | None = None
    target_delta: float | None = None
    target_epsilon: float | None = None
    noise_multiplier: float | None = None
    expected_steps_per_epoch: int | None = None
    expected_batch_size: float | None = None
    total_steps: int | None = None
    mechanism_kind: str | None = None
    is_horizon_process: bool = False
    calibration_source: str | None = None
    horizon_process_state: dict | None = None
    mf_n_steps: int | None = None
    mf_min_sep: int | None = None
    mf_max_participations: int | None = None
    lr_scheduler: str | None = None
    learning_rate: float | None = None
    warmup_steps: int | None = None
    lr_scheduler_kwargs: dict | None = None
    sampler_stream_key: dict | None = None        # {"seed", "impl"}, before the per-rank fold


def checkpoint_dir(output_dir: str, step: int) -> str:
    return os.path.join(output_dir, f"{PREFIX}-{step}")


def list_checkpoints(output_dir: str) -> list[str]:
    if not os.path.isdir(output_dir):
        return []
    found = []
    for name in os.listdir(output_dir):
        m = re.fullmatch(rf"{PREFIX}-(\d+)", name)
        if m and os.path.isdir(os.path.join(output_dir, name)):
            found.append((int(m.group(1)), os.path.join(output_dir, name)))
    return [p for _, p in sorted(found)]


def latest_checkpoint(output_dir: str) -> str | None:
    ckpts = list_checkpoints(output_dir)
    return ckpts[-1] if ckpts else None


def rotate_checkpoints(output_dir: str, limit: int | None, keep: str | None = None) -> list[str]:
    """Deletes the oldest checkpoints beyond ``limit`` (never ``keep``, the best model). Returns what was removed."""
    if limit is None or limit <= 0:
        return []
    ckpts = list_checkpoints(output_dir)
    removable = [c for c in ckpts if keep is None or os.path.abspath(c) != os.path.abspath(keep)]
    excess = len(ckpts) - limit
    removed = []
    for c in removable[:max(0, excess)]:
        shutil.rmtree(c, ignore_errors=True)
        removed.append(c)
    return removed


_REFERENCE_MODULE = "opake.api.transformers.trainer._checkpoint"


class _ReferenceAlias:
    """While active, ``opake.api.transformers.trainer._checkpoint.RuntimeCheckpoint`` resolves to this package's
    ``RuntimeCheckpoint``. The reference pickles its bundle as an instance of that dataclass
    (``trainer/_checkpoint.py:313-389``), so a ``dp_state.pt`` is portable in both directions only if that class path
    can be pickled and unpickled here. Nothing is registered when a real ``opake`` distribution is importable."""

    def __enter__(self):
        import importlib.util
        import sys
        import types

        self._added: list[str] = []
        self._names = None
        try:
            real = importlib.util.find_spec(_REFERENCE_MODULE) is not None
        except (ImportError, ValueError):
            real = False
        if real:
            return self
        parts = _REFERENCE_MODULE.split(".")
        for i in range(1, len(parts) + 1):
            name = ".".join(parts[:i])
            if name not in sys.modules:
                mod = types.ModuleType(name)
                mod.__path__ = []          # a package, so that sub-module lookups consult sys.modules
                sys.modules[name] = mod
                self._added.append(name)
        sys.modules[_REFERENCE_MODULE].RuntimeCheckpoint = RuntimeCheckpoint
        self._names = (RuntimeCheckpoint.__module__, RuntimeCheckpoint.__qualname__)
        RuntimeCheckpoint.__module__, RuntimeCheckpoint.__qualname__ = _REFERENCE_MODULE, "RuntimeCheckpoint"
        return self

    def __exit__(self, *exc):
        import sys

        if self._names is not None:
            RuntimeCheckpoint.__module__, RuntimeCheckpoint.__qualname__ = self._names
        for name in reversed(self._added):
            sys.modules.pop(name, None)
        return False


def save_runtime(path: str, rt: RuntimeCheckpoint) -> None:
    """Writes ``dp_state.pt`` as the reference does: a pickled ``RuntimeCheckpoint`` instance under the reference's
    class path, so either implementation can resume from the file."""
    with _ReferenceAlias() as alias:
        if alias._names is None:        # the reference itself is importable: hand it a plain mapping-free instance of its class
            import importlib

            ref_cls = importlib.import_module(_REFERENCE_MODULE).RuntimeCheckpoint
            names = {f.name for f in dataclasses.fields(ref_cls)}
            torch.save(ref_cls(**{k: v for k, v in dataclasses.asdict(rt).items() if k in names}), path)
        else:
            torch.save(rt, path)


def load_runtime(path: str) -> RuntimeCheckpoint:
    try:
        with _ReferenceAlias():
            raw = torch.load(path, map_location="cpu", weights_only=False)
    except Exception as e:
        raise CheckpointError(f"cannot read DP runtime state {path}: {e}") from e
    if dataclasses.is_dataclass(raw) and not isinstance(raw, type):
        raw = {f.name: getattr(raw, f.name) for f in dataclasses.fields(raw)}
    if not isinstance(raw, dict) or "version" not in raw:
        raise CheckpointError(f"{path} is not a DP runtime bundle")
    if raw["version"] != BUNDLE_VERSION:
        raise CheckpointError(f"{path} has bundle version {raw['version']}, this build reads version {BUNDLE_VERSION}")
    names = {f.name for f in dataclasses.fields(RuntimeCheckpoint)}
    return RuntimeCheckpoint(**{k: v for k, v in raw.items() if k in names})


def _differs(a, b) -> bool:
    if isinstance(a, float) or isinstance(b, float):
        if a is None or b is None:
            return a is not b
        return abs(float(a) - float(b)) > 1e-12 * max(1.0, abs(float(a)), abs(float(b)))
    return a != b


def compare_runtime(saved: RuntimeCheckpoint, now: RuntimeCheckpoint) -> None:
    """Applies the drift rules between a checkpoint and the freshly configured run."""
    strict = saved.is_horizon_process or (saved.mechanism_kind or "").startswith("mf_")
    for name in DP_RELEVANT:
        a, b = getattr(saved, name), getattr(now, name)
        if a is not None and b is not None and _differs(a, b):
            msg = (f"resume changes the privacy-relevant setting {name}: checkpoint {a!r}, now {b!r}")
            if strict:
                raise CheckpointError(msg + "; a horizon-calibrated or matrix-factorisation run cannot change it mid-way")
            warnings.warn(msg + "; the accountant continues with the new value", stacklevel=3)
    if saved.total_steps is not None and now.total_steps is not None and saved.total_steps != now.total_steps:
        if strict or now.total_steps < saved.total_steps and saved.mechanism_kind != "gaussian":
            raise CheckpointError(f"resume changes total_steps from {saved.total_steps} to {now.total_steps}, which the "
                                  "checkpointed noise calibration does not cover")
        warnings.warn(f"total_steps changed from {saved.total_steps} to {now.total_steps}: the privacy spend is "
                      "re-evaluated for the new length", stacklevel=3)
    for name in SHAPE:
        a, b = getattr(saved, name), getattr(now, name)
        if a is not None and b is not None and _differs(a, b):
            warnings.warn(f"resume changes {name} from {a!r} to {b!r} (learning-rate shape only)", stacklevel=3)


def save_rng_state(path: str) -> None:
    state: dict[str, Any] = {"python": random.getstate(), "numpy": np.random.get_state(), "cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state_all()
    torch.save(state, path)


def load_rng_state(path: str) -> bool:
    if not os.path.exists(path):
        return False
    state = torch.load(path, map_location="cpu", weights_only=False)
    random.setstate(state["python"])
    np.random.set_state(state["numpy"])
    torch.set_rng_state(state["cpu"])
    if "cuda" in state and torch.cuda.is_available():
        try:
            torch.cuda.set_rng_state_all(state["cuda"])
        except Exception:
            warnings.warn("CUDA RNG state of the checkpoint does not match the visible devices; not restored", stacklevel=2)
    return True
