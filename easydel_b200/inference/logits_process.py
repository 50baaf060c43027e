"""Logits processors and warpers for ``generate()`` (easydel/inference/logits_process.py): the Hugging Face style
list API over torch tensors. The serving engine does not use these; its penalties / top-k / top-p / min-p run in
the fused sampler kernel."""

from __future__ import annotations

import math
import typing as tp

import torch


class LogitsProcessor:
    def __call__(self, input_ids: torch.Tensor, scores: torch.Tensor, cur_len: int) -> torch.Tensor:
        raise NotImplementedError


LogitsWarper = LogitsProcessor


class LogitsProcessorList(list):
    def __call__(self, input_ids, scores, cur_len: int = 0):
        for p in self:
            scores = p(input_ids, scores, cur_len)
        return scores


class TemperatureLogitsWarper(LogitsProcessor):
    def __init__(self, temperature: float):
        if temperature <= 0:
            raise ValueError("temperature must be positive")
        self.t = temperature

    def __call__(self, input_ids, scores, cur_len=0):
        return scores / self.t


class TopKLogitsWarper(LogitsProcessor):
    def __init__(self, top_k: int, filter_value: float = -float("inf"), min_tokens_to_keep: int = 1):
        self.k, self.fill = max(top_k, min_tokens_to_keep), filter_value

    def __call__(self, input_ids, scores, cur_len=0):
        k = min(self.k, scores.shape[-1])
        kth = scores.topk(k, -1).values[..., -1:]
        return scores.masked_fill(scores < kth, self.fill)


class TopPLogitsWarper(LogitsProcessor):
    def __init__(self, top_p: float, filter_value: float = -float("inf"), min_tokens_to_keep: int = 1):
        self.p, self.fill, self.keep = top_p, filter_value, min_tokens_to_keep

    def __call__(self, input_ids, scores, cur_len=0):
        s, idx = scores.sort(-1, descending=True)
        cum = s.softmax(-1).cumsum(-1)
        remove = cum - s.softmax(-1) > self.p
        remove[..., : self.keep] = False
        return scores.masked_fill(torch.zeros_like(remove).scatter(-1, idx, remove), self.fill)


class MinPLogitsWarper(LogitsProcessor):
    def __init__(self, min_p: float, filter_value: float = -float("inf")):
        self.p, self.fill = min_p, filter_value

    def __call__(self, input_ids, scores, cur_len=0):
        probs = scores.softmax(-1)
        return scores.masked_fill(probs < self.p * probs.max(-1, keepdim=True).values, self.fill)


class RepetitionPenaltyLogitsProcessor(LogitsProcessor):
    def __init__(self, penalty: float):
        self.penalty = penalty

    def __call__(self, input_ids, scores, cur_len=0):
        picked = scores.gather(-1, input_ids)
        picked = torch.where(picked < 0, picked * self.penalty, picked / self.penalty)
        return scores.scatter(-1, input_ids, picked)


class PresencePenaltyLogitsProcessor(LogitsProcessor):
    def __init__(self, penalty: float):
        self.penalty = penalty

    def __call__(self, input_ids, scores, cur_len=0):
        seen = torch.zeros_like(scores, dtype=torch.bool).scatter(-1, input_ids, True)
        return scores - self.penalty * seen


class FrequencyPenaltyLogitsProcessor(LogitsProcessor):
    def __init__(self, penalty: float):
        self.penalty = penalty

    def __call__(self, input_ids, scores, cur_len=0):
        counts = torch.zeros_like(scores).scatter_add(-1, input_ids, torch.ones_like(input_ids, dtype=scores.dtype))
        return scores - self.penalty * counts


class MinLengthLogitsProcessor(LogitsProcessor):
    def __init__(self, min_length: int, eos_token_id: int | tp.Sequence[int]):
        self.n = min_length
        self.eos = [eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id)

    def __call__(self, input_ids, scores, cur_len=0):
        if cur_len < self.n:
            scores = scores.clone()
            scores[..., self.eos] = -float("inf")
        return scores


class ForcedBOSTokenLogitsProcessor(LogitsProcessor):
    def __init__(self, bos_token_id: int):
        self.bos = bos_token_id

    def __call__(self, input_ids, scores, cur_len=0):
        if cur_len == 1:
            out = torch.full_like(scores, -float("inf"))
            out[..., self.bos] = 0
            return out
        return scores


class ForcedEOSTokenLogitsProcessor(LogitsProcessor):
    def __init__(self, max_length: int, eos_token_id: int):
        self.max_length, self.eos = max_length, eos_token_id

    def __call__(self, input_ids, scores, cur_len=0):
        if cur_len == self.max_length - 1:
            out = torch.full_like(scores, -float("inf"))
            out[..., self.eos] = 0
            return out
        return scores


class SuppressTokensLogitsProcessor(LogitsProcessor):
    def __init__(self, suppress_tokens: tp.Sequence[int]):
        self.tokens = list(suppress_tokens)

    def __call__(self, input_ids, scores, cur_len=0):
        scores = scores.clone()
        scores[..., self.tokens] = -float("inf")
        return scores


class SuppressTokensAtBeginLogitsProcessor(SuppressTokensLogitsProcessor):
    def __init__(self, begin_suppress_tokens, begin_index: int):
        super().__init__(begin_suppress_tokens)
        self.begin = begin_index

    def __call__(self, input_ids, scores, cur_len=0):
        return super().__call__(input_ids, scores, cur_len) if cur_len == self.begin else scores


class NoRepeatNGramLogitsProcessor(LogitsProcessor):
    def __init__(self, ngram_size: int):
        self.n = ngram_size

    def __call__(self, input_ids, scores, cur_len=0):
        n = self.n
        if input_ids.shape[1] + 1 < n:
            return scores
        scores = scores.clone()
        for b, row in enumerate(input_ids.tolist()):
            prefix = tuple(row[len(row) - n + 1:]) if n > 1 else ()
            for i in range(len(row) - n + 1):
                if tuple(row[i:i + n - 1]) == prefix:
                    scores[b, row[i + n - 1]] = -float("inf")
        return scores


class LogitBiasProcessor(LogitsProcessor):
    def __init__(self, bias: dict[int, float]):
        self.ids = list(bias)
        self.vals = list(bias.values())

    def __call__(self, input_ids, scores, cur_len=0):
        scores = scores.clone()
        scores[..., self.ids] += torch.tensor(self.vals, dtype=scores.dtype, device=scores.device)
        return scores


class AllowedTokensLogitsProcessor(LogitsProcessor):
    def __init__(self, allowed: tp.Sequence[int]):
        self.allowed = list(allowed)

    def __call__(self, input_ids, scores, cur_len=0):
        out = torch.full_like(scores, -float("inf"))
        out[..., self.allowed] = scores[..., self.allowed]
        return out


def processors_from_sampling_params(sp, eos_token_id=None) -> LogitsProcessorList:
    """The processor list equivalent to a ``SamplingParams`` (order: penalties, bias / masks, warpers)."""
    ps = LogitsProcessorList()
    if sp.repetition_penalty != 1.0:
        ps.append(RepetitionPenaltyLogitsProcessor(sp.repetition_penalty))
    if sp.presence_penalty:
        ps.append(PresencePenaltyLogitsProcessor(sp.presence_penalty))
    if sp.frequency_penalty:
        ps.append(FrequencyPenaltyLogitsProcessor(sp.frequency_penalty))
    if sp.logit_bias:
        ps.append(LogitBiasProcessor(sp.logit_bias))
    if sp.allowed_token_ids:
        ps.append(AllowedTokensLogitsProcessor(sp.allowed_token_ids))
    if sp.min_tokens and eos_token_id is not None:
        ps.append(MinLengthLogitsProcessor(sp.min_tokens, eos_token_id))
    if sp.temperature not in (0.0, 1.0):
        ps.append(TemperatureLogitsWarper(sp.temperature))
    if sp.top_k:
        ps.append(TopKLogitsWarper(sp.top_k))
    if sp.top_p < 1.0:
        ps.append(TopPLogitsWarper(sp.top_p))
    if sp.min_p > 0.0:
        ps.append(MinPLogitsWarper(sp.min_p))
    return ps
