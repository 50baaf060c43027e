"""Whisper transcription pipeline: audio front end, long-form inference, OpenAI-compatible server."""

from .audio import chunk_iter, load_audio, log_mel_spectrogram, mel_filter_bank
from .config import vWhisperInferenceConfig
from .core import merge_token_overlap, vWhisperInference

__all__ = ["chunk_iter", "load_audio", "log_mel_spectrogram", "mel_filter_bank", "merge_token_overlap",
           "vWhisperInference", "vWhisperInferenceConfig"]
