"""Settings of the Whisper transcription pipeline (easydel/inference/vwhisper/config.py:63-172)."""

from __future__ import annotations

import dataclasses
import typing as tp


@dataclasses.dataclass(frozen=True)
class vWhisperInferenceConfig:
    """``None`` fields fall back to the model's generation config (or the default given in the comment)."""

    batch_size: int | None = 1                  # 30-second windows decoded together
    max_length: int | None = None               # decoder positions per window (model: max_target_positions)
    generation_config: tp.Any = None            # a Hugging Face GenerationConfig (lang_to_id, task_to_id, ...)
    logits_processor: tp.Any = None
    return_timestamps: bool | None = None       # False
    task: str | None = None                     # "transcribe" | "translate"
    language: str | None = None                 # "en", "<|en|>", "english"; None = no language token forced
    is_multilingual: bool | None = None

    def replace(self, **kw) -> "vWhisperInferenceConfig":
        return dataclasses.replace(self, **{k: v for k, v in kw.items() if v is not None})
