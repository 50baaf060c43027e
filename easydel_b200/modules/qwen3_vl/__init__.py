from .modeling_qwen3_vl import (Qwen3VLConfig, Qwen3VLForConditionalGeneration, Qwen3VLMoeConfig,
                                Qwen3VLMoeForConditionalGeneration, Qwen3VLVisionConfig, Qwen3VLVisionTransformer)

__all__ = ["Qwen3VLConfig", "Qwen3VLForConditionalGeneration", "Qwen3VLMoeConfig",
           "Qwen3VLMoeForConditionalGeneration", "Qwen3VLVisionConfig", "Qwen3VLVisionTransformer"]
