"""``TrainingArguments``: every knob of a training run, JSON round-trippable.

Field names and defaults follow easydel/trainers/training_configurations.py:222-793 (optimizer
``adamw``, scheduler ``none``, lr 5e-5, weight decay 0.01, ``total_batch_size`` 32, accumulation 1,
10 epochs, ``resume_if_possible``, ``save_optimizer_state``, ``do_last_save``...). Fields that only
make sense for a tracing compiler or TPUs are accepted and ignored so that configs port unchanged.
"""

from __future__ import annotations

import dataclasses
import json
import os
import re
import typing as tp
from dataclasses import dataclass, field

from ..infra.base_config import TRAINING_ARGS_NAME
from ..infra.loss_utils import LossConfig
from ..optimizers import OptimizerFactory, SchedulerConfig
from ..infra.factory import registry as _registry  # noqa: F401

_TRAINER_ARGS: dict[str, type] = {}
_TRAINERS: dict[str, type] = {}


def register_trainer_arguments(name: str):
    def deco(cls):
        _TRAINER_ARGS[name] = cls
        cls.trainer_type = name
        return cls

    return deco


def register_trainer(name: str):
    def deco(cls):
        _TRAINERS[name] = cls
        cls.trainer_type = name
        return cls

    return deco


def get_trainer_class(name: str):
    from .. import trainers as _t  # noqa: F401  (registers everything)

    return _TRAINERS[name]


def get_trainer_arguments_class(name: str):
    from .. import trainers as _t  # noqa: F401

    return _TRAINER_ARGS[name]


def parse_time_limit(s: str | float | int | None) -> float | None:
    """``"90min"``, ``"2h"``, ``"45s"``, ``"1d"`` or a number of seconds."""
    if s is None:
        return None
    if isinstance(s, (int, float)):
        return float(s)
    m = re.fullmatch(r"\s*([\d.]+)\s*(s|sec|m|min|h|hr|d)?\s*", str(s).lower())
    if not m:
        raise ValueError(f"cannot parse time limit {s!r}")
    mult = {None: 1, "s": 1, "sec": 1, "m": 60, "min": 60, "h": 3600, "hr": 3600, "d": 86400}[m.group(2)]
    return float(m.group(1)) * mult


@register_trainer_arguments("base")
@dataclass
class TrainingArguments:
    auto_shard_states: bool = True
    aux_loss_enabled: bool = False
    backend: str | None = None
    clip_grad: float | None = None
    custom_scheduler: tp.Callable[[int], tp.Any] | None = None
    dataloader_num_workers: int | None = 0
    dataloader_pin_memory: bool | None = True
    do_eval: bool = False
    do_last_save: bool = True
    do_train: bool = True
    eval_batch_size: int | None = None
    evaluation_steps: int | None = None
    extra_optimizer_kwargs: dict | None = None
    frozen_parameters: str | None = None
    gradient_accumulation_steps: int = 1
    ids_to_pop_from_dataset: list[str] | None = None
    is_fine_tuning: bool = True
    init_tx: bool = True
    learning_rate: float = 5e-5
    learning_rate_end: float | None = None
    log_all_workers: bool = False
    log_grad_norms: bool = True
    report_metrics: bool = True
    log_steps: int = 10
    loss_config: LossConfig | dict | None = None
    lmhead_chunksize: int | None = None
    low_mem_usage: bool = True
    max_evaluation_steps: int | None = None
    max_length: int | None = 4096
    max_training_steps: int | None = None
    per_epoch_training_steps: int | None = None
    per_epoch_evaluation_steps: int | None = None
    model_name: str | None = None
    model_parameters: dict | None = None
    metrics_to_show_in_rich_pbar: list[str] | None = None
    generation_top_p: float | None = None
    generation_top_k: int | None = None
    generation_temperature: float | None = None
    generation_do_sample: bool | None = None
    generation_max_new_tokens: int | None = None
    generation_interval: int | None = None
    generation_prompts: list = field(default_factory=list)
    generation_seed: int | None = None
    benchmark_interval: int | None = None
    benchmark_tasks: list | None = None          # lm-eval task names run every ``benchmark_interval`` steps
    benchmark_limit: int | None = None
    preemption_signals: tuple = ("SIGTERM", "SIGUSR1")   # signals that trigger a checkpoint and a clean stop
    use_esurge_generation: bool = True
    esurge_hbm_utilization: float | None = None
    esurge_max_num_seqs: int | None = None
    esurge_page_size: int | None = None
    esurge_max_num_batched_tokens: int | None = None
    esurge_enable_prefix_caching: bool | None = None
    num_train_epochs: int = 10
    offload_dataset: bool = False
    optimizer: str = "adamw"
    performance_mode: bool = False
    process_zero_is_admin: bool = True
    progress_bar_type: str = "tqdm"
    remove_ckpt_after_load: bool = False
    remove_unused_columns: bool = True
    report_steps: int = 5
    save_interval_minutes: float | None = None
    save_directory: str | None = "EasyDeL-Checkpoints"
    save_optimizer_state: bool = True
    merge_lora_before_save: bool = True
    save_steps: int | None = None
    save_total_limit: int | None = None
    save_tpu_preemption_checkpoints: bool = True
    scheduler: str = "none"
    shuffle_seed_train: int = 64871
    step_start_point: int | None = None
    force_step_start_point: bool = False
    resume_if_possible: bool = True
    shuffle_train_dataset: bool = True
    total_batch_size: int = 32
    training_time_limit: str | None = None
    train_on_inputs: bool = True
    trainer_prefix: str | None = None
    truncation_mode: str = "keep_end"
    tx_mu_dtype: tp.Any = None
    track_memory: bool | float = False
    use_data_collator: bool = True
    use_grain: bool = True
    use_wandb: bool = True
    verbose: bool = True
    wandb_entity: str | None = None
    wandb_name: str | None = None
    warmup_steps: int = 0
    weight_decay: float = 0.01
    watchers: list = field(default_factory=list)
    weight_distribution_pattern: str = r".*"
    weight_distribution_log_steps: int = 0
    step_partition_spec: tp.Any = (("dp", "fsdp"), "sp")
    jax_distributed_config: dict | None = None
    sparsify_module: bool = False
    sparse_module_type: str = "bcoo"
    state_apply_fn_kwarguments_to_model: dict | None = None
    quantization_mode: str | None = None
    quantization_group_size: int | None = None
    quantization_bits: int | None = None
    pruning_module: tp.Any = None
    max_sequence_length: dataclasses.InitVar[int | None] = None

    trainer_type: tp.ClassVar[str] = "base"

    def __post_init__(self, max_sequence_length=None):
        if max_sequence_length is not None:
            self.max_length = max_sequence_length
        if self.gradient_accumulation_steps < 1:
            raise ValueError("gradient_accumulation_steps must be >= 1")
        if isinstance(self.loss_config, dict):
            self.loss_config = LossConfig(**self.loss_config)
        if self.model_name is None:
            self.model_name = "easydel-model"
        self.optimizer = str(getattr(self.optimizer, "value", self.optimizer))
        self.scheduler = str(getattr(self.scheduler, "value", self.scheduler))
        self._time_limit_s = parse_time_limit(self.training_time_limit)
        self._setup_optimizer()

    # ------------------------------------------------------------------ optimizer
    def _setup_optimizer(self) -> None:
        extra = self.extra_optimizer_kwargs or {}
        self.optimizer_kwargs = {
            "learning_rate": self.learning_rate, "learning_rate_end": self.learning_rate_end,
            "optimizer": self.optimizer, "scheduler": self.scheduler, "warmup_steps": self.warmup_steps,
            "gradient_accumulation_steps": self.gradient_accumulation_steps, "weight_decay": self.weight_decay,
            "steps": self.max_training_steps, "clip_grad": self.clip_grad, "mu_dtype": self.tx_mu_dtype, **extra,
        }

    def get_optimizer_and_scheduler(self, steps: int | None = None):
        kw = dict(self.optimizer_kwargs)
        kw["steps"] = steps or kw["steps"]
        sched = kw.pop("scheduler", None)
        if sched in ("none", None):
            sched = None
        cfg = SchedulerConfig(scheduler_type=sched, steps=kw.pop("steps"), learning_rate=kw.pop("learning_rate"),
                              learning_rate_end=kw.pop("learning_rate_end"), warmup_steps=kw.pop("warmup_steps"),
                              exponent=kw.pop("exponent", 1))
        kw.pop("gradient_accumulation_steps", None)
        return OptimizerFactory.create(optimizer_type=kw.pop("optimizer"), scheduler_config=cfg,
                                       clip_grad=kw.pop("clip_grad"), weight_decay=kw.pop("weight_decay"),
                                       custom_scheduler=self.custom_scheduler, **kw)

    def get_tx_template(self):
        """An optimizer built without a step count: enough to rebuild the state layout on resume."""
        return self.get_optimizer_and_scheduler(self.max_training_steps or 1)[0]

    # ------------------------------------------------------------------ paths
    def get_path(self) -> str:
        return os.path.join(self.save_directory or ".", self.model_name or "model")

    def step_directory(self, step: int) -> str:
        return os.path.join(self.get_path(), f"run-{step}")

    @property
    def is_process_zero(self) -> bool:
        return int(os.environ.get("RANK", "0")) == 0

    @property
    def can_log_metrics(self) -> bool:
        return self.report_metrics and (self.is_process_zero or self.log_all_workers)

    @property
    def training_time_seconds(self) -> float | None:
        return self._time_limit_s

    # ------------------------------------------------------------------ (de)serialisation
    def to_dict(self) -> dict:
        out = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            if callable(v) and not isinstance(v, type):
                continue
            if isinstance(v, LossConfig):
                v = v.to_dict()
            if isinstance(v, tuple):
                v = _tuple_to_list(v)
            out[f.name] = v
        out["trainer_config_class"] = type(self).__name__
        out["trainer_type"] = type(self).trainer_type
        return out

    @classmethod
    def from_dict(cls, d: dict):
        d = dict(d)
        d.pop("trainer_config_class", None)
        ttype = d.pop("trainer_type", None)
        target = cls
        if cls is TrainingArguments and ttype in _TRAINER_ARGS:
            target = _TRAINER_ARGS[ttype]
        names = {f.name for f in dataclasses.fields(target)} | {"max_sequence_length"}
        return target(**{k: v for k, v in d.items() if k in names})

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True, default=str) + "\n"

    def save_arguments(self, path: str | os.PathLike) -> str:
        p = str(path)
        if os.path.isdir(p):
            p = os.path.join(p, TRAINING_ARGS_NAME)
        tmp = p + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            f.write(self.to_json_string())
        os.replace(tmp, p)
        return p

    @classmethod
    def load_arguments(cls, path: str | os.PathLike):
        p = str(path)
        if os.path.isdir(p):
            p = os.path.join(p, TRAINING_ARGS_NAME)
        with open(p, encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    load_from_json = load_arguments
    save_to_json = save_arguments


def _tuple_to_list(v):
    return [_tuple_to_list(x) if isinstance(x, tuple) else x for x in v]
