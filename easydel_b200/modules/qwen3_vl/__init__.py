from .modeling_qwen3_vl import (Qwen3_5Config, Qwen3_5ForConditionalGeneration, Qwen3_5MoeConfig,
                                Qwen3_5MoeForConditionalGeneration, Qwen3_5VisionConfig, Qwen3VLConfig,
                                Qwen3VLForConditionalGeneration, Qwen3VLMoeConfig,
                                Qwen3VLMoeForConditionalGeneration, Qwen3VLVisionConfig, Qwen3VLVisionTransformer)

__all__ = ["Qwen3_5Config", "Qwen3_5ForConditionalGeneration", "Qwen3_5MoeConfig",
           "Qwen3_5MoeForConditionalGeneration", "Qwen3_5VisionConfig", "Qwen3VLConfig",
           "Qwen3VLForConditionalGeneration", "Qwen3VLMoeConfig",
           "Qwen3VLMoeForConditionalGeneration", "Qwen3VLVisionConfig", "Qwen3VLVisionTransformer"]
