from .configuration import LlamaConfig
from .modeling import LlamaForCausalLM, LlamaForSequenceClassification, LlamaModel

__all__ = ["LlamaConfig", "LlamaForCausalLM", "LlamaForSequenceClassification", "LlamaModel"]
