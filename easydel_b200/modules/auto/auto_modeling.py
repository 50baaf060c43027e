"""Auto classes: pick config / model class from ``config.json`` (easydel/modules/auto/*, 1425 LoC).

``AutoEasyDeLModelForCausalLM.from_pretrained`` accepts an EasyDeL checkpoint directory (zarr
layout), a Hugging Face safetensors directory, or a training directory with ``run-*`` checkpoints.
The twelve ``AutoEasyDeLModel*`` classes differ only in the task they look up; each has an
``AutoState*`` twin returning an ``EasyDeLState``.
"""

from __future__ import annotations

import json
import os
import typing as tp

import torch

from ...infra.base_config import CONFIG_NAME
from ...infra.factory import TaskType, _ensure_models_imported, registry


def _read_model_type(path: str) -> tuple[str, list[str] | None]:
    from ...io.checkpoint import _resolve_dir

    path = _resolve_dir(path)
    with open(os.path.join(path, CONFIG_NAME), encoding="utf-8") as f:
        d = json.load(f)
    return d["model_type"], d.get("architectures")


def resolve_model_class(path: str, task: TaskType = TaskType.CAUSAL_LM):
    _ensure_models_imported()
    mtype, _ = _read_model_type(path)
    return registry.get_module_registration(task, mtype).module


class AutoEasyDeLConfig:
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, sharding_axis_dims=None, sharding_axis_names=None,
                        partition_axis=None, backend=None, platform=None, model_task: TaskType = TaskType.CAUSAL_LM,
                        from_torch: bool = False, **kwargs):
        from ...io.checkpoint import _resolve_dir, load_config

        return load_config(_resolve_dir(pretrained_model_name_or_path), kwargs or None,
                           sharding_axis_dims=sharding_axis_dims, sharding_axis_names=sharding_axis_names,
                           partition_axis=partition_axis)


class AutoShardAndGatherFunctions:
    """Returns per-parameter placement callables. With the explicit runtime these are identity / gather
    closures over the mesh; kept so code written against the reference's loader API keeps working."""

    @classmethod
    def from_config(cls, config, partition_rules=None, flatten: bool = True, model_task=TaskType.CAUSAL_LM, **_):
        shard = lambda t: t  # noqa: E731
        gather = lambda t: t  # noqa: E731
        return shard, gather

    from_pretrained = from_config


class BaseAutoEasyModel:
    model_task: TaskType = TaskType.CAUSAL_LM

    @classmethod
    def from_config(cls, config, dtype=torch.bfloat16, param_dtype=None, **kw):
        _ensure_models_imported()
        mod = registry.get_module_registration(cls.model_task, config.model_type).module
        return mod(config, dtype=dtype, param_dtype=param_dtype or dtype)

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, **kwargs):
        model_cls = resolve_model_class(pretrained_model_name_or_path, cls.model_task)
        return model_cls.from_pretrained(pretrained_model_name_or_path, **kwargs)


class BaseAutoEasyState:
    model_task: TaskType = TaskType.CAUSAL_LM

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, **kwargs):
        model_cls = resolve_model_class(pretrained_model_name_or_path, cls.model_task)
        return model_cls.from_pretrained(pretrained_model_name_or_path, **kwargs).to_state()


def _mk(name: str, task: TaskType, base):
    return type(name, (base,), {"model_task": task, "__doc__": f"Auto class for task ``{task.value}``."})


_TASKS = {
    "ForCausalLM": TaskType.CAUSAL_LM,
    "ForSequenceClassification": TaskType.SEQUENCE_CLASSIFICATION,
    "ForImageTextToText": TaskType.IMAGE_TEXT_TO_TEXT,
    "ForSeq2SeqLM": TaskType.SEQUENCE_TO_SEQUENCE,
    "ForSpeechSeq2Seq": TaskType.SPEECH_SEQUENCE_TO_SEQUENCE,
    "ForZeroShotImageClassification": TaskType.ZERO_SHOT_IMAGE_CLASSIFICATION,
    "ForDiffusionLM": TaskType.DIFFUSION_LM,
    "ForImageClassification": TaskType.IMAGE_CLASSIFICATION,
    "ForAudioClassification": TaskType.AUDIO_CLASSIFICATION,
    "ForEmbedding": TaskType.EMBEDDING,
    "ForAnyToAny": TaskType.ANY_TO_ANY,
}

AutoEasyDeLModel = _mk("AutoEasyDeLModel", TaskType.BASE_MODULE, BaseAutoEasyModel)
AutoEasyDeLVisionModel = _mk("AutoEasyDeLVisionModel", TaskType.BASE_VISION, BaseAutoEasyModel)
AutoState = _mk("AutoState", TaskType.BASE_MODULE, BaseAutoEasyState)
AutoStateVisionModel = _mk("AutoStateVisionModel", TaskType.BASE_VISION, BaseAutoEasyState)
__all__ = ["AutoEasyDeLConfig", "AutoShardAndGatherFunctions", "AutoEasyDeLModel", "AutoEasyDeLVisionModel",
           "AutoState", "AutoStateVisionModel", "resolve_model_class", "BaseAutoEasyModel", "BaseAutoEasyState"]
for _suffix, _task in _TASKS.items():
    globals()[f"AutoEasyDeLModel{_suffix}"] = _mk(f"AutoEasyDeLModel{_suffix}", _task, BaseAutoEasyModel)
    globals()[f"AutoState{_suffix}"] = _mk(f"AutoState{_suffix}", _task, BaseAutoEasyState)
    __all__ += [f"AutoEasyDeLModel{_suffix}", f"AutoState{_suffix}"]

# the reference's spelling of the any-to-any auto class
AutoEasyDeLAnyToAnyModel = globals()["AutoEasyDeLModelForAnyToAny"]
AutoStateAnyToAnyModel = globals()["AutoStateForAnyToAny"]
__all__ += ["AutoEasyDeLAnyToAnyModel", "AutoStateAnyToAnyModel"]
