"""Trainers. Importing this package registers every trainer type."""

from .base_trainer import BaseTrainer, Trainer, TrainerOutput, find_latest_checkpoint
from .metrics import LogWatcher, StepMetrics
from .training_configurations import (TrainingArguments, get_trainer_arguments_class, get_trainer_class,
                                      register_trainer, register_trainer_arguments)

register_trainer("base")(Trainer)

__all__ = ["BaseTrainer", "Trainer", "TrainerOutput", "TrainingArguments", "LogWatcher", "StepMetrics",
           "find_latest_checkpoint", "get_trainer_class", "get_trainer_arguments_class"]
