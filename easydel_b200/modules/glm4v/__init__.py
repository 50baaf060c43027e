from .modeling_glm4v import (Glm46VConfig, Glm46VForConditionalGeneration, Glm4vConfig, Glm4vForConditionalGeneration,
                             Glm4vMoeConfig, Glm4vMoeForConditionalGeneration, Glm4vVisionConfig,
                             Glm4vVisionTransformer)

__all__ = ["Glm46VConfig", "Glm46VForConditionalGeneration", "Glm4vConfig", "Glm4vForConditionalGeneration",
           "Glm4vMoeConfig", "Glm4vMoeForConditionalGeneration", "Glm4vVisionConfig", "Glm4vVisionTransformer"]
