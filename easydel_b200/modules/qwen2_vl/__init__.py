from .modeling_qwen2_vl import (Qwen2VLConfig, Qwen2VLForConditionalGeneration, Qwen2VLVisionConfig,
                                Qwen2VLVisionTransformer, mrope_positions)

__all__ = ["Qwen2VLConfig", "Qwen2VLForConditionalGeneration", "Qwen2VLVisionConfig", "Qwen2VLVisionTransformer",
           "mrope_positions"]
