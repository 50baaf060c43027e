"""Model / config registry keyed by task type and ``model_type`` string.

Same contract as easydel/infra/factory.py:92-689: ``register_config("llama")``
decorates a config class, ``register_module(TaskType.CAUSAL_LM, config=...,
model_type="llama")`` decorates a module class, and the auto classes look both
up by the ``model_type`` found in ``config.json``.
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass, field

from .etils import StrEnum


class TaskType(StrEnum):
    CAUSAL_LM = "causal-language-model"
    VISION_LM = "vision-language-model"
    DIFFUSION_LM = "diffusion-language-model"
    IMAGE_TEXT_TO_TEXT = "image-text-to-text"
    BASE_MODULE = "base-module"
    BASE_VISION = "vision-module"
    SEQUENCE_TO_SEQUENCE = "sequence-to-sequence"
    SPEECH_SEQUENCE_TO_SEQUENCE = "speech-sequence-to-sequence"
    ZERO_SHOT_IMAGE_CLASSIFICATION = "zero-shot-image-classification"
    SEQUENCE_CLASSIFICATION = "sequence-classification"
    AUDIO_CLASSIFICATION = "audio-classification"
    IMAGE_CLASSIFICATION = "image-classification"
    EMBEDDING = "embedding"
    ANY_TO_ANY = "any-to-any"
    AUTO_BIND = "auto-bind"


class ConfigType(StrEnum):
    MODULE_CONFIG = "module-config"


@dataclass
class ModuleRegistration:
    module: type
    config: type
    embedding_layer_names: list[str] | None = None
    layernorm_names: list[str] | None = None


@dataclass
class Registry:
    _configs: dict[str, dict[str, type]] = field(default_factory=lambda: {ConfigType.MODULE_CONFIG.value: {}})
    _modules: dict[str, dict[str, ModuleRegistration]] = field(default_factory=dict)

    def register_config(self, config_type: str, config_field: ConfigType = ConfigType.MODULE_CONFIG):
        def deco(cls):
            self._configs.setdefault(str(config_field), {})[config_type] = cls
            cls.model_type = getattr(cls, "model_type", None) or config_type
            return cls

        return deco

    def register_module(self, task_type: TaskType | str, config: type, model_type: str,
                        embedding_layer_names: list[str] | None = None, layernorm_names: list[str] | None = None):
        def deco(cls):
            self._modules.setdefault(str(TaskType(task_type)), {})[model_type] = ModuleRegistration(
                module=cls, config=config, embedding_layer_names=embedding_layer_names,
                layernorm_names=layernorm_names)
            cls._model_task = str(TaskType(task_type))
            cls._model_type = model_type
            cls.config_class = config
            return cls

        return deco

    def get_config(self, config_type: str, config_field: ConfigType = ConfigType.MODULE_CONFIG) -> type:
        try:
            return self._configs[str(config_field)][config_type]
        except KeyError:
            raise KeyError(f"config type {config_type!r} is not registered; known: "
                           f"{sorted(self._configs[str(config_field)])}") from None

    def get_module_registration(self, task_type: TaskType | str, model_type: str) -> ModuleRegistration:
        task = str(TaskType(task_type))
        try:
            return self._modules[task][model_type]
        except KeyError:
            known = sorted(self._modules.get(task, {}))
            raise KeyError(f"no {task} module registered for model_type {model_type!r}; known: {known}") from None

    def alias(self, alias: str, target: str) -> None:
        """Makes ``alias`` resolve to everything registered as ``target``: composite checkpoints name their halves
        with their own model types (``qwen3_vl_text``, ``glm4v_moe_vision``...) although the classes are shared."""
        cfgs = self._configs[ConfigType.MODULE_CONFIG.value]
        if target not in cfgs:
            raise KeyError(f"cannot alias {alias!r}: config type {target!r} is not registered")
        cfgs.setdefault(alias, cfgs[target])
        for table in self._modules.values():
            if target in table:
                table.setdefault(alias, table[target])

    @property
    def task_registry(self) -> dict[str, dict[str, ModuleRegistration]]:
        return self._modules

    @property
    def config_registry(self) -> dict[str, type]:
        return self._configs[ConfigType.MODULE_CONFIG.value]


registry = Registry()
register_config = registry.register_config
register_module = registry.register_module


def get_modules_by_type(model_type: str, task_type: TaskType | str = TaskType.CAUSAL_LM):
    """Returns (config class, module class) for a model type, as easydel.modules.auto does."""
    _ensure_models_imported()
    reg = registry.get_module_registration(task_type, model_type)
    return reg.config, reg.module


def _ensure_models_imported() -> None:
    from .. import modules  # noqa: F401  (importing the package registers every family)
