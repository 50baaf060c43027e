from .clip import (CLIPConfig, CLIPModel, CLIPTextConfig, SiglipConfig, SiglipModel,  # noqa: F401
                   SiglipTextConfig)
from .vit import (CLIPVisionConfig, CLIPVisionModel, SiglipVisionConfig, SiglipVisionModel,  # noqa: F401
                  VisionTransformer)

__all__ = ["CLIPConfig", "CLIPModel", "CLIPTextConfig", "CLIPVisionConfig", "CLIPVisionModel", "SiglipConfig",
           "SiglipModel", "SiglipTextConfig", "SiglipVisionConfig", "SiglipVisionModel", "VisionTransformer"]
