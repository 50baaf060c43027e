from .modeling_llama4 import (Llama4Config, Llama4ForConditionalGeneration, Llama4MultiModalProjector,  # noqa: F401
                              Llama4VisionConfig, Llama4VisionModel, pixel_shuffle)

__all__ = ["Llama4Config", "Llama4ForConditionalGeneration", "Llama4MultiModalProjector", "Llama4VisionConfig",
           "Llama4VisionModel", "pixel_shuffle"]
