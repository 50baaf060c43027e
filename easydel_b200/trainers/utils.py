"""Collators and batch helpers (the basics of easydel/trainers/utils.py)."""

from __future__ import annotations

import typing as tp

import numpy as np
import torch


def _as_tensor(v):
    if isinstance(v, torch.Tensor):
        return v
    if isinstance(v, np.ndarray):
        return torch.from_numpy(v)
    return torch.as_tensor(v)


def pad_to_length(t: torch.Tensor, length: int, pad_value, left: bool = False) -> torch.Tensor:
    if t.shape[-1] >= length:
        return t
    pad = torch.full((*t.shape[:-1], length - t.shape[-1]), pad_value, dtype=t.dtype)
    return torch.cat([pad, t], dim=-1) if left else torch.cat([t, pad], dim=-1)


def default_collate(features: list[dict], pad_token_id: int = 0, max_length: int | None = None,
                    truncation_mode: str = "keep_end", label_pad: int = -100) -> dict[str, torch.Tensor]:
    """Stacks a list of example dicts. Ragged 1-D fields are right-padded: ids with ``pad_token_id``,
    ``labels`` with ``-100``, masks / segment ids with 0. Over-long rows are truncated per ``truncation_mode``."""
    out: dict[str, torch.Tensor] = {}
    keys = [k for k in features[0].keys() if features[0][k] is not None]
    for k in keys:
        vals = [_as_tensor(f[k]) for f in features]
        if vals[0].dim() == 0:
            out[k] = torch.stack(vals)
            continue
        if max_length is not None and vals[0].dim() == 1:
            vals = [(v[-max_length:] if truncation_mode == "keep_end" else v[:max_length]) for v in vals]
        L = max(v.shape[-1] for v in vals)
        if any(v.shape[-1] != L for v in vals):
            pv = label_pad if k == "labels" else (pad_token_id if "input_ids" in k else 0)
            vals = [pad_to_length(v, L, pv) for v in vals]
        out[k] = torch.stack(vals)
    return out


class DataCollatorForCompletionOnlyLM:
    """Masks everything before the response template with ``-100`` (completion-only loss)."""

    def __init__(self, tokenizer, response_template: str | list[int], instruction_template=None, ignore_index=-100):
        self.tokenizer = tokenizer
        self.ignore_index = ignore_index
        self.response_ids = tokenizer.encode(response_template, add_special_tokens=False) \
            if isinstance(response_template, str) else list(response_template)

    def __call__(self, features: list[dict]) -> dict[str, torch.Tensor]:
        batch = default_collate(features, pad_token_id=getattr(self.tokenizer, "pad_token_id", 0) or 0)
        labels = batch["input_ids"].clone()
        n = len(self.response_ids)
        for i, row in enumerate(batch["input_ids"].tolist()):
            start = None
            for j in range(len(row) - n + 1):
                if row[j:j + n] == self.response_ids:
                    start = j + n
            if start is None:
                labels[i, :] = self.ignore_index
            else:
                labels[i, :start] = self.ignore_index
        if "attention_mask" in batch:
            labels[batch["attention_mask"] == 0] = self.ignore_index
        batch["labels"] = labels
        return batch
