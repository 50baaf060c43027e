"""easydel_b200: a Blackwell-native (sm_100a) LLM training and serving framework with EasyDeL's surface."""

__version__ = "0.1.0"

import importlib as _importlib
import typing as _tp

_LAZY: dict[str, str] = {
    # infra
    "EasyDeLBaseConfig": "easydel_b200.infra.base_config", "EasyDeLBaseConfigDict": "easydel_b200.infra.base_config",
    "PartitionAxis": "easydel_b200.infra.base_config",
    "EasyDeLBaseModule": "easydel_b200.infra.base_module", "EasyDeLState": "easydel_b200.infra.base_state",
    "LossConfig": "easydel_b200.infra.loss_utils", "LossMetrics": "easydel_b200.infra.loss_utils",
    "TaskType": "easydel_b200.infra.factory", "ConfigType": "easydel_b200.infra.factory",
    "register_config": "easydel_b200.infra.factory", "register_module": "easydel_b200.infra.factory",
    "get_modules_by_type": "easydel_b200.infra.factory",
    "EasyDeLOptimizers": "easydel_b200.infra.etils", "EasyDeLSchedulers": "easydel_b200.infra.etils",
    "EasyDeLGradientCheckPointers": "easydel_b200.infra.etils", "AttentionMechanisms": "easydel_b200.infra.etils",
    "EasyDeLRuntimeError": "easydel_b200.infra.errors", "EasyDeLSyntaxRuntimeError": "easydel_b200.infra.errors",
    "EasyDeLTimerError": "easydel_b200.infra.errors", "EasyDeLBackends": "easydel_b200.infra.etils",
    "EasyDeLPlatforms": "easydel_b200.infra.etils", "MoEMethods": "easydel_b200.infra.etils",
    "Registry": "easydel_b200.infra.factory",
    "ModelConverter": "easydel_b200.utils.parameters_transformation",
    "StateDictConverter": "easydel_b200.utils.parameters_transformation",
    "TensorConverter": "easydel_b200.utils.parameters_transformation",
    # trainers
    "TrainingArguments": "easydel_b200.trainers", "Trainer": "easydel_b200.trainers",
    "BaseTrainer": "easydel_b200.trainers", "TrainerOutput": "easydel_b200.trainers",
    "LogWatcher": "easydel_b200.trainers",
    # models
    "LlamaConfig": "easydel_b200.modules.llama", "LlamaModel": "easydel_b200.modules.llama",
    "LlamaForCausalLM": "easydel_b200.modules.llama",
    "LlamaForSequenceClassification": "easydel_b200.modules.llama",
    # serving
    "eSurge": "easydel_b200.inference.esurge", "eSurgeApiServer": "easydel_b200.inference.esurge.server",
    "InferenceApiRouter": "easydel_b200.inference.oai_proxies",
    "ToolParserManager": "easydel_b200.inference.tools.parsers",
    "ToolParser": "easydel_b200.inference.tools.parsers",
    "AttentionModule": "easydel_b200.layers.attention",
    "EngineRequest": "easydel_b200.inference.esurge.scheduler",
    "EngineRequestStatus": "easydel_b200.inference.esurge.scheduler",
    "ResponsesStreamBuilder": "easydel_b200.inference.stream_protocol",
    "eSurgeLMEvalAdapter": "easydel_b200.inference.evaluations.esurge_eval",
    "MultiModalManager": "easydel_b200.inference.esurge.multimodal",
    # quantisation
    "EasyDeLQuantizationConfig": "easydel_b200.layers.quantization",
    "QuantizationType": "easydel_b200.layers.quantization", "EasyQuantizer": "easydel_b200.layers.quantization",
    "TurboQuantConfig": "easydel_b200.layers.turboquant", "TurboQuantConstants": "easydel_b200.layers.turboquant",
    # speech
    "vWhisperInference": "easydel_b200.inference.vwhisper",
    "vWhisperInferenceConfig": "easydel_b200.inference.vwhisper",
}


_LAZY.update({_n: "easydel_b200.ops.registry" for _n in (
    "OperationMetadata", "BaseOperationConfig", "AttentionConfig", "FlashAttentionConfig",
    "BlockSparseAttentionConfig", "ScaledDotProductAttentionConfig", "RingAttentionConfig", "RaggedPageAttentionv2Config",
    "RaggedPageAttentionv3Config", "AttentionOutput", "OperationRegistry", "OperationImpl",
    "FlashAttn", "BlockSparseAttn", "VanillaAttn", "ScaledDotProductAttn",
    "RingAttn", "RaggedPageAttnV2", "RaggedPageAttnV3", "PagedFlashAttn",
    "AutoRegressiveDecodeAttn", "FlexibleAttentionModule")})


def _register_lazy(names: dict[str, str]) -> None:
    _LAZY.update(names)


# Packages searched (in order) for public names that are not listed above: every model family, trainer,
# serving class and data helper is reachable as ``easydel_b200.<Name>`` like in the reference's flat namespace.
_SEARCH = ("modules", "trainers", "inference", "data", "optimizers", "layers", "caching", "parallel", "utils", "elarge")


def __getattr__(name: str) -> _tp.Any:
    if name.startswith("__"):
        raise AttributeError(name)
    if name in _LAZY:
        return getattr(_importlib.import_module(_LAZY[name]), name)
    try:
        return _importlib.import_module(f"{__name__}.{name}")
    except ModuleNotFoundError as e:
        if e.name != f"{__name__}.{name}":
            raise
    for pkg in _SEARCH:
        try:
            mod = _importlib.import_module(f"{__name__}.{pkg}")
        except ModuleNotFoundError:
            continue
        if name in getattr(mod, "__dict__", {}):
            return mod.__dict__[name]
    raise AttributeError(f"module 'easydel_b200' has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
