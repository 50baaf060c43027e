"""Trainers. Importing this package registers every trainer type."""

from .base_trainer import BaseTrainer, Trainer, TrainerOutput, find_latest_checkpoint
from .metrics import LogWatcher, StepMetrics
from .training_configurations import (TrainingArguments, get_trainer_arguments_class, get_trainer_class,
                                      register_trainer, register_trainer_arguments)

register_trainer("base")(Trainer)
register_trainer("trainer")(Trainer)

from .sft import SFTConfig, SFTTrainer  # noqa: E402
from .preference import (BCOConfig, BCOTrainer, CPOConfig, CPOTrainer, DPOConfig, DPODataCollator,  # noqa: E402
                         DPOTrainer, KTOConfig, KTOTrainer, ORPOConfig, ORPOTrainer, RewardConfig, RewardTrainer,
                         dpo_loss)
from .rl import (GFPOConfig, GFPOTrainer, GRPOConfig, GRPOTrainer, GSPOConfig, GSPOTrainer, RLVRConfig,  # noqa: E402
                 RLVRTrainer, SDPOConfig, SDPOTrainer, MathVerifier, FormatVerifier, LengthPenaltyVerifier,
                 CodeExecutionVerifier)
from .rl_online import (NashMDConfig, NashMDTrainer, PPOConfig, PPOTrainer, XPOConfig, XPOTrainer)  # noqa: E402
from .distillation import (DistillationConfig, DistillationTrainer, GKDConfig, GKDTrainer,  # noqa: E402
                           OnPolicyDistillationConfig, OnPolicyDistillationTrainer, SeqKDConfig, SeqKDTrainer,
                           SparseDistillationConfig, SparseDistillationTrainer)
from .embedding import EmbeddingConfig, EmbeddingTrainer  # noqa: E402
from .agentic import (AgenticMoshPitConfig, AgenticMoshPitTrainer, EnvironmentManager, TextEnvironment,  # noqa: E402
                      ToolEnvironment)
from .ray_dist import RayDistributedConfig, RayDistributedTrainer  # noqa: E402

register_trainer("ray_dist")(RayDistributedTrainer)

from . import prompt_transforms  # noqa: E402,F401
from .prompt_transforms import *  # noqa: E402,F401,F403

__all__ = [n for n in dir() if not n.startswith("_")]
