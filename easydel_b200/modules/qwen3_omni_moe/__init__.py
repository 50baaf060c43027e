from .modeling_qwen3_omni_moe import (Qwen3OmniMoeAudioEncoder, Qwen3OmniMoeAudioEncoderConfig, Qwen3OmniMoeConfig,
                                      Qwen3OmniMoeForConditionalGeneration, Qwen3OmniMoeThinkerConfig,
                                      Qwen3OmniMoeThinkerForConditionalGeneration, audio_output_lengths)
from .speech import (Qwen3OmniMoeCode2Wav, Qwen3OmniMoeCode2WavConfig, Qwen3OmniMoeTalkerCodePredictor,
                     Qwen3OmniMoeTalkerCodePredictorConfig, Qwen3OmniMoeTalkerConfig,
                     Qwen3OmniMoeTalkerForConditionalGeneration, Qwen3OmniMoeTalkerTextConfig, SpeechTokenIds,
                     talker_inputs)

__all__ = ["Qwen3OmniMoeAudioEncoder", "Qwen3OmniMoeAudioEncoderConfig", "Qwen3OmniMoeConfig",
           "Qwen3OmniMoeForConditionalGeneration", "Qwen3OmniMoeThinkerConfig",
           "Qwen3OmniMoeThinkerForConditionalGeneration", "audio_output_lengths", "Qwen3OmniMoeCode2Wav",
           "Qwen3OmniMoeCode2WavConfig", "Qwen3OmniMoeTalkerCodePredictor", "Qwen3OmniMoeTalkerCodePredictorConfig",
           "Qwen3OmniMoeTalkerConfig", "Qwen3OmniMoeTalkerForConditionalGeneration", "Qwen3OmniMoeTalkerTextConfig",
           "SpeechTokenIds", "talker_inputs"]
