from .modeling_qwen3_omni_moe import (Qwen3OmniMoeAudioEncoder, Qwen3OmniMoeAudioEncoderConfig, Qwen3OmniMoeConfig,
                                      Qwen3OmniMoeForConditionalGeneration, Qwen3OmniMoeThinkerConfig,
                                      Qwen3OmniMoeThinkerForConditionalGeneration, audio_output_lengths)

__all__ = ["Qwen3OmniMoeAudioEncoder", "Qwen3OmniMoeAudioEncoderConfig", "Qwen3OmniMoeConfig",
           "Qwen3OmniMoeForConditionalGeneration", "Qwen3OmniMoeThinkerConfig",
           "Qwen3OmniMoeThinkerForConditionalGeneration", "audio_output_lengths"]
