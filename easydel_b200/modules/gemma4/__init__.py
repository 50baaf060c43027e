from .modeling_gemma4 import Gemma4Cache, Gemma4ForCausalLM, Gemma4TextConfig, Gemma4TextModel

__all__ = ["Gemma4Cache", "Gemma4ForCausalLM", "Gemma4TextConfig", "Gemma4TextModel"]
