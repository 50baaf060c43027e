from .modeling_llava import LlavaConfig, LlavaForConditionalGeneration  # noqa: F401

__all__ = ["LlavaConfig", "LlavaForConditionalGeneration"]
