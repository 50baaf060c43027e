from .modeling_gemma4 import (Gemma4Cache, Gemma4Config, Gemma4ForCausalLM, Gemma4ForConditionalGeneration,
                              Gemma4TextConfig, Gemma4TextModel, Gemma4VisionConfig, Gemma4VisionModel)

__all__ = ["Gemma4Cache", "Gemma4Config", "Gemma4ForCausalLM", "Gemma4ForConditionalGeneration", "Gemma4TextConfig",
           "Gemma4TextModel", "Gemma4VisionConfig", "Gemma4VisionModel"]
