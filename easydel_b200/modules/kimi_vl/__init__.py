from .modeling_kimi_vl import (KimiVLConfig, KimiVLForConditionalGeneration, KimiVLMultiModalProjector, MoonViTConfig,
                               MoonVitPretrainedModel)

__all__ = ["KimiVLConfig", "KimiVLForConditionalGeneration", "KimiVLMultiModalProjector", "MoonViTConfig",
           "MoonVitPretrainedModel"]
