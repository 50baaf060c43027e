from .modeling_aya_vision import AyaVisionConfig, AyaVisionForConditionalGeneration, AyaVisionMultiModalProjector

__all__ = ["AyaVisionConfig", "AyaVisionForConditionalGeneration", "AyaVisionMultiModalProjector"]
