"""Trainer layer: ``DPTrainer``, ``TrainingArguments`` and the TRL-shaped ``SFTTrainer`` / ``DPOTrainer``
(counterpart of ``opake.transformers``, packages/opake-transformers/src/opake/transformers/__init__.py)."""
from .callback import (BestModelSaveCallback, EarlyStoppingCallback, JsonlLoggerCallback, PrinterCallback, TensorBoardCallback,
                       TrainerCallback, WandbCallback)
from .dp_trainer import DPTrainer, TrainOutput
from .state import DPTrainerState, TrainerControl
from .training_arguments import TrainingArguments

__all__ = ["DPTrainer", "TrainOutput", "TrainingArguments", "DPTrainerState", "TrainerControl", "TrainerCallback",
           "PrinterCallback", "JsonlLoggerCallback", "TensorBoardCallback", "WandbCallback", "BestModelSaveCallback",
           "EarlyStoppingCallback", "SFTTrainer", "SFTConfig", "DPOTrainer", "DPOConfig", "trl"]


def __getattr__(name):
    if name == "trl":
        import importlib

        return importlib.import_module(".trl", __name__)
    if name in ("SFTTrainer", "SFTConfig"):
        from .trl import sft_trainer as m
        return getattr(m, name)
    if name in ("DPOTrainer", "DPOConfig"):
        from .trl import dpo_trainer as m
        return getattr(m, name)
    raise AttributeError(name)
