from .vit import (CLIPVisionConfig, CLIPVisionModel, SiglipVisionConfig, SiglipVisionModel,  # noqa: F401
                  VisionTransformer)

__all__ = ["CLIPVisionConfig", "CLIPVisionModel", "SiglipVisionConfig", "SiglipVisionModel", "VisionTransformer"]
