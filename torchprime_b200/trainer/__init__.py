"""Trainer registry keyed by ``task.name`` (reference: trainer/__init__.py:6-9)."""

from .base_trainer import Trainer
from .sft_trainer import SFTTrainer

TRAINERS = {"train": Trainer, "sft": SFTTrainer}

__all__ = ["Trainer", "SFTTrainer", "TRAINERS"]
