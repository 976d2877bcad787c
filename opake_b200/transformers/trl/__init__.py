"""TRL-shaped trainers on top of ``DPTrainer``."""
from .dpo_trainer import DPOConfig, DPOTrainer
from .sft_trainer import SFTConfig, SFTTrainer

__all__ = ["SFTTrainer", "SFTConfig", "DPOTrainer", "DPOConfig"]
