from .modeling_whisper import (
    WhisperConfig,
    WhisperForAudioClassification,
    WhisperForConditionalGeneration,
    WhisperModel,
    shift_tokens_right,
    sinusoids,
)

__all__ = ["WhisperConfig", "WhisperForAudioClassification", "WhisperForConditionalGeneration", "WhisperModel",
           "shift_tokens_right", "sinusoids"]
