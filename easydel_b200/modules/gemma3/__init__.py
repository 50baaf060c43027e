from .modeling_gemma3 import Gemma3Config, Gemma3ForConditionalGeneration, Gemma3MultiModalProjector

__all__ = ["Gemma3Config", "Gemma3ForConditionalGeneration", "Gemma3MultiModalProjector"]
