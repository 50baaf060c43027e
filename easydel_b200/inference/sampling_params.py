"""Sampling parameters (easydel/inference/sampling_params.py:474-516, BeamSearchParams :755)."""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    n: int = 1
    best_of: int | None = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    min_p: float = 0.0
    top_k: int = 0
    seed: int | None = None
    stop: str | list[str] | None = None
    stop_token_ids: list[int] | None = None
    stop_pattern: str | None = None
    bad_words: list[str] | None = None
    ignore_eos: bool = False
    max_tokens: int | None = 16
    min_tokens: int = 0
    logprobs: int | None = None
    prompt_logprobs: int | None = None
    detokenize: bool = True
    skip_special_tokens: bool = True
    spaces_between_special_tokens: bool = True
    include_stop_str_in_output: bool = False
    logit_bias: dict[int, float] | None = None
    allowed_token_ids: list[int] | None = None
    guided_decoding: tp.Any = None
    extra_args: dict | None = None

    def __post_init__(self):
        if self.n < 1:
            raise ValueError("n must be at least 1")
        if self.best_of is not None and self.best_of < self.n:
            raise ValueError("best_of must be >= n")
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if self.top_k < -1:
            raise ValueError("top_k must be -1 (disabled), 0 (disabled) or positive")
        if self.top_k == -1:
            self.top_k = 0
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if not -2.0 <= self.presence_penalty <= 2.0 or not -2.0 <= self.frequency_penalty <= 2.0:
            raise ValueError("presence / frequency penalties must be in [-2, 2]")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.min_tokens < 0 or (self.max_tokens is not None and self.min_tokens > self.max_tokens):
            raise ValueError("min_tokens must be in [0, max_tokens]")
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        self.stop = list(self.stop or [])
        self.stop_token_ids = list(self.stop_token_ids or [])

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1

    @property
    def needs_penalties(self) -> bool:
        return self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.repetition_penalty != 1.0

    def clone(self, **kw) -> "SamplingParams":
        import dataclasses

        return dataclasses.replace(self, **kw)


@dataclass
class JitableSamplingParams:
    """Array-friendly subset (the reference's ``JitableSamplingParams`` :194-210)."""

    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0

    @classmethod
    def from_sampling_params(cls, sp: SamplingParams) -> "JitableSamplingParams":
        return cls(sp.temperature, sp.top_p, sp.top_k, sp.min_p, sp.presence_penalty, sp.frequency_penalty,
                   sp.repetition_penalty)


@dataclass
class BeamSearchParams:
    beam_width: int = 4
    max_tokens: int = 16
    ignore_eos: bool = False
    temperature: float = 0.0
    length_penalty: float = 1.0
    include_stop_str_in_output: bool = False
