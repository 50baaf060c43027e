"""Supervised fine-tuning trainer (easydel/trainers/supervised_fine_tuning_trainer/sft_trainer.py:46-267).

The base trainer already runs the causal-LM step; this class adds what the reference's ``SFTTrainer`` adds
in front of it: turning raw text / chat examples into token rows, completion-only or assistant-only label
masks (``labels = -100`` outside the answer) and sequence packing into fixed-length rows with segment ids.
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass

import torch

from .base_trainer import Trainer
from .packer import pack_sequences
from .training_configurations import TrainingArguments, register_trainer, register_trainer_arguments


@register_trainer_arguments("sft")
@dataclass
class SFTConfig(TrainingArguments):
    trainer_prefix: str | None = "sfttrainer"
    dataset_text_field: str | None = "text"
    add_special_tokens: bool = False
    packing: bool = False
    packing_strategy: str = "bfd"          # bfd (first-fit decreasing) | wrapped (greedy concatenation)
    completion_only_loss: bool | None = None
    assistant_only_loss: bool = False
    dataset_num_proc: int | None = None
    eval_packing: bool | None = None
    formatting_func: tp.Callable | None = None


def _tokenize_example(ex: dict, tok, args: SFTConfig) -> dict:
    """One raw example -> ``input_ids`` (+ ``completion_mask`` / ``assistant_masks`` when derivable)."""
    if "input_ids" in ex:
        return ex
    if args.formatting_func is not None:
        ex = {"text": args.formatting_func(ex)}
    max_len = args.max_length
    if "messages" in ex or "conversations" in ex:
        msgs = ex.get("messages") or ex.get("conversations")
        full = tok.apply_chat_template(msgs, tokenize=True, add_generation_prompt=False)
        ids = list(full["input_ids"] if isinstance(full, dict) else full)
        mask = [0] * len(ids)
        if args.assistant_only_loss:
            # tokens contributed by assistant turns: difference between prefixes that end before / after the turn
            for i, m in enumerate(msgs):
                if m.get("role") != "assistant":
                    continue
                pre = tok.apply_chat_template(msgs[:i], tokenize=True, add_generation_prompt=True) if i else []
                upto = tok.apply_chat_template(msgs[:i + 1], tokenize=True, add_generation_prompt=False)
                pre = list(pre["input_ids"] if isinstance(pre, dict) else pre)
                upto = list(upto["input_ids"] if isinstance(upto, dict) else upto)
                for j in range(len(pre), min(len(upto), len(ids))):
                    mask[j] = 1
        out = {"input_ids": ids[:max_len]}
        if args.assistant_only_loss:
            out["assistant_masks"] = mask[:max_len]
        return out
    if "prompt" in ex and "completion" in ex:
        p = tok(ex["prompt"], add_special_tokens=args.add_special_tokens)["input_ids"]
        c = tok(ex["completion"], add_special_tokens=False)["input_ids"]
        eos = getattr(tok, "eos_token_id", None)
        if eos is not None and (not c or c[-1] != eos):
            c = c + [eos]
        ids = (p + c)[:max_len]
        return {"input_ids": ids, "completion_mask": ([0] * len(p) + [1] * len(c))[:max_len]}
    text = ex[args.dataset_text_field or "text"]
    ids = tok(text, add_special_tokens=args.add_special_tokens, truncation=max_len is not None,
              max_length=max_len)["input_ids"]
    return {"input_ids": list(ids)}


def _with_labels(row: dict, args: SFTConfig) -> dict:
    ids = list(row["input_ids"])
    labels = list(ids)
    use_completion = args.completion_only_loss if args.completion_only_loss is not None else "completion_mask" in row
    if use_completion and "completion_mask" in row:
        labels = [t if m else -100 for t, m in zip(ids, row["completion_mask"])]
    if args.assistant_only_loss and "assistant_masks" in row:
        labels = [t if m else -100 for t, m in zip(labels, row["assistant_masks"])]
    out = {"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels}
    return out


class _MappedDataset:
    def __init__(self, rows: list[dict]):
        self.rows = rows

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]


@register_trainer("sft")
class SFTTrainer(Trainer):
    trainer_type = "sft"
    arguments_class = SFTConfig

    def __init__(self, arguments: SFTConfig | None = None, model=None, processing_class=None, train_dataset=None,
                 eval_dataset=None, formatting_func=None, data_collator=None, **kw):
        arguments = arguments or SFTConfig()
        if formatting_func is not None:
            arguments.formatting_func = formatting_func
        train_dataset = kw.pop("dataset_train", train_dataset)
        eval_dataset = kw.pop("dataset_eval", eval_dataset)
        tok = processing_class if processing_class is not None else kw.get("tokenizer")
        if train_dataset is not None:
            train_dataset = self._prepare(train_dataset, tok, arguments, arguments.packing)
        if eval_dataset is not None:
            pack_eval = arguments.packing if arguments.eval_packing is None else arguments.eval_packing
            eval_dataset = self._prepare(eval_dataset, tok, arguments, pack_eval)
        super().__init__(arguments=arguments, model=model, dataset_train=train_dataset, dataset_eval=eval_dataset,
                         data_collator=data_collator, processing_class=tok, **kw)

    @staticmethod
    def _prepare(dataset, tok, args: SFTConfig, packing: bool):
        try:
            first = dataset[0]
        except Exception:
            return dataset    # streaming source: assumed tokenised already
        if "input_ids" in first and "labels" in first and not packing:
            return dataset
        if "input_ids" not in first and tok is None:
            raise ValueError("SFTTrainer needs `processing_class` to tokenise raw text datasets")
        rows = [_with_labels(_tokenize_example(dict(dataset[i]), tok, args), args) for i in range(len(dataset))]
        if packing:
            if args.max_length is None:
                raise ValueError("packing requires `max_length`")
            rows = pack_sequences(rows, args.max_length, strategy=args.packing_strategy,
                                  pad_token_id=(getattr(tok, "pad_token_id", None) or 0))
        return _MappedDataset(rows)
