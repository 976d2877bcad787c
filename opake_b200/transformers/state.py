"""Trainer bookkeeping that is saved as ``trainer_state.json`` (packages/opake-transformers/src/opake/api/
transformers/trainer/_state.py:39-124): the Hugging Face ``TrainerState`` fields plus the privacy spend."""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any

__all__ = ["DPTrainerState", "TrainerControl"]


@dataclass
class DPTrainerState:
    epoch: float | None = None
    global_step: int = 0
    max_steps: int = 0
    logging_steps: int = 500
    eval_steps: int | None = None
    save_steps: int = 500
    train_batch_size: int | None = None
    num_train_epochs: int = 0
    num_input_tokens_seen: int = 0
    total_flos: float = 0.0
    log_history: list = field(default_factory=list)
    best_metric: float | None = None
    best_global_step: int | None = None
    best_model_checkpoint: str | None = None
    is_local_process_zero: bool = True
    is_world_process_zero: bool = True
    stateful_callbacks: dict = field(default_factory=dict)
    # privacy bookkeeping
    privacy_epsilon: float | None = None
    privacy_target_epsilon_reached: bool = False      # stop-at-epsilon ended the run before max_steps
    privacy_delta: float | None = None
    noise_multiplier: float | None = None
    sample_rate: float | None = None
    examples_seen: int = 0
    clipped_fraction: float | None = None
    # distributed run description
    world_size: int = 1
    ddp_backend: str | None = None

    def save_to_json(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            f.write(json.dumps(dataclasses.asdict(self), indent=2, sort_keys=True, default=_jsonable) + "\n")

    @classmethod
    def load_from_json(cls, path: str) -> "DPTrainerState":
        with open(path, encoding="utf-8") as f:
            raw = json.load(f)
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in raw.items() if k in names})


def _jsonable(x: Any):
    if hasattr(x, "item"):
        return x.item()
    if hasattr(x, "tolist"):
        return x.tolist()
    return str(x)


@dataclass
class TrainerControl:
    """Flags a callback may raise to steer the loop (same names as the Hugging Face control object)."""
    should_training_stop: bool = False
    should_epoch_stop: bool = False
    should_save: bool = False
    should_evaluate: bool = False
    should_log: bool = False

    def _new_step(self):
        self.should_save = self.should_evaluate = self.should_log = False

    def _new_epoch(self):
        self.should_epoch_stop = False
