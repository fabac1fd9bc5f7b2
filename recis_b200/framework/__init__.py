from .checkpoint_manager import CheckpointManager, Saver
from .trainer import Trainer, TrainingArguments

__all__ = ["Trainer", "TrainingArguments", "CheckpointManager", "Saver"]
