"""Per-example preprocessing for the trainers: raw text / chat / preference examples -> the token rows the
collators take (easydel/trainers/prompt_transforms.py:75-1300).

Every transform is a callable ``example -> row`` (or ``-> list[row]`` for :class:`BCOPreprocessTransform`, which
expands a pair into two unpaired rows), usable with ``data.transforms.MappedSource`` or a plain ``map``. Chat-format
fields (lists of ``{"role", "content"}``) go through the tokenizer's chat template; the prompt of a preference pair
is the common prefix of the two conversations when it is not given.

    SFT         input_ids (+ completion_mask / assistant_masks)
    DPO / ORPO  prompt_input_ids, chosen_input_ids, rejected_input_ids
    CPO         = DPO rows
    KTO / BCO   prompt_input_ids, completion_input_ids, label
    Reward      input_ids_chosen, input_ids_rejected (+ margin)
    GRPO / PPO  prompt_input_ids (left-truncated) + every other field kept for the reward functions
    Embedding   query_input_ids, positive_input_ids (+ negative_input_ids)
"""

from __future__ import annotations

import typing as tp


def _ids(x) -> list[int]:
    return list(x["input_ids"] if isinstance(x, dict) or hasattr(x, "keys") else x)


def purify_example(example: dict, keep_fields: set[str] | None = None) -> dict:
    """Drops ``None`` values and, with ``keep_fields``, everything not listed."""
    return {k: v for k, v in example.items() if v is not None and (keep_fields is None or k in keep_fields)}


def is_conversational(value) -> bool:
    return isinstance(value, list) and bool(value) and isinstance(value[0], dict) and "role" in value[0]


def extract_prompt_from_preference(example: dict) -> dict:
    """``chosen`` / ``rejected`` conversations without a ``prompt``: the shared leading turns become the prompt."""
    if "prompt" in example and example["prompt"] is not None:
        return example
    c, r = example["chosen"], example["rejected"]
    if not (is_conversational(c) and is_conversational(r)):
        return dict(example, prompt="")
    n = 0
    while n < min(len(c), len(r)) - 1 and c[n] == r[n]:
        n += 1
    return dict(example, prompt=c[:n], chosen=c[n:], rejected=r[n:])


def apply_chat_template_to_preference(example: dict, tokenizer, tools=None) -> dict:
    """Renders conversational ``prompt`` / ``chosen`` / ``rejected`` / ``completion`` fields to text; the completion
    text is what the template adds after the rendered prompt."""
    out = dict(example)
    prompt = example.get("prompt")
    if not is_conversational(prompt):
        return out
    kw = {"tools": tools} if tools else {}
    p_text = tokenizer.apply_chat_template(prompt, tokenize=False, add_generation_prompt=True, **kw)
    out["prompt"] = p_text
    for key in ("chosen", "rejected", "completion"):
        val = example.get(key)
        if is_conversational(val):
            full = tokenizer.apply_chat_template(prompt + val, tokenize=False, add_generation_prompt=False, **kw)
            out[key] = full[len(p_text):] if full.startswith(p_text) else "".join(m.get("content") or "" for m in val)
    return out


class Transform:
    """Base class: holds the tokenizer and the length limits."""

    def __init__(self, tokenizer, max_prompt_length: int | None = None, max_completion_length: int | None = None,
                 max_length: int | None = None, tools=None, add_eos: bool = True):
        self.tok, self.mp, self.mc, self.max_length = tokenizer, max_prompt_length, max_completion_length, max_length
        self.tools, self.add_eos = tools, add_eos

    def _prompt(self, text: str) -> list[int]:
        ids = _ids(self.tok(text, add_special_tokens=True))
        return ids[-self.mp:] if self.mp else ids                 # prompts keep their end

    def _completion(self, text: str) -> list[int]:
        ids = _ids(self.tok(text, add_special_tokens=False))
        eos = getattr(self.tok, "eos_token_id", None)
        if self.add_eos and eos is not None and (not ids or ids[-1] != eos):
            ids = ids + [eos]
        return ids[: self.mc] if self.mc else ids                 # completions keep their beginning

    def __call__(self, example: dict):
        raise NotImplementedError


class ExpandTransform(Transform):
    """A transform that returns a list of rows per example."""


class SFTPreprocessTransform(Transform):
    def __init__(self, tokenizer, max_length: int | None = None, dataset_text_field: str = "text",
                 formatting_func: tp.Callable | None = None, assistant_only_loss: bool = False,
                 add_special_tokens: bool = True, **kw):
        super().__init__(tokenizer, max_length=max_length, **kw)
        from .sft import SFTConfig

        self.args = SFTConfig(max_length=max_length, dataset_text_field=dataset_text_field,
                              formatting_func=formatting_func, assistant_only_loss=assistant_only_loss,
                              add_special_tokens=add_special_tokens)

    def __call__(self, example: dict) -> dict:
        from .sft import _tokenize_example

        return _tokenize_example(purify_example(example), self.tok, self.args)


class DPOPreprocessTransform(Transform):
    def __call__(self, example: dict) -> dict:
        ex = apply_chat_template_to_preference(extract_prompt_from_preference(purify_example(example)), self.tok,
                                               self.tools)
        row = {"prompt_input_ids": self._prompt(ex["prompt"]), "chosen_input_ids": self._completion(ex["chosen"]),
               "rejected_input_ids": self._completion(ex["rejected"])}
        for k in ("reference_chosen_logps", "reference_rejected_logps", "margin"):
            if k in ex:
                row[k] = ex[k]
        return row


class ORPOPreprocessTransform(DPOPreprocessTransform):
    pass


class CPOPreprocessTransform(DPOPreprocessTransform):
    pass


class KTOPreprocessTransform(Transform):
    """``prompt`` + ``completion`` + ``label`` rows; a pair (``chosen`` / ``rejected``) is taken as its chosen half
    unless ``label`` says otherwise."""

    def __call__(self, example: dict) -> dict:
        ex = purify_example(example)
        if "completion" not in ex and "chosen" in ex:
            good = bool(ex.get("label", True))
            ex = dict(extract_prompt_from_preference(ex))
            ex["completion"], ex["label"] = (ex["chosen"] if good else ex["rejected"]), good
        ex = apply_chat_template_to_preference(ex, self.tok, self.tools)
        return {"prompt_input_ids": self._prompt(ex["prompt"]),
                "completion_input_ids": self._completion(ex["completion"]), "label": bool(ex.get("label", True))}


class BCOPreprocessTransform(ExpandTransform):
    """A preference pair becomes two unpaired rows (chosen = desirable, rejected = undesirable); an unpaired example
    passes through as one row."""

    def __call__(self, example: dict) -> list[dict]:
        ex = purify_example(example)
        one = KTOPreprocessTransform(self.tok, self.mp, self.mc, self.max_length, self.tools, self.add_eos)
        if "chosen" in ex and "rejected" in ex and "completion" not in ex:
            return [one(dict(ex, label=True)), one(dict(ex, label=False))]
        return [one(ex)]


class RewardPreprocessTransform(Transform):
    def __call__(self, example: dict) -> dict:
        ex = apply_chat_template_to_preference(extract_prompt_from_preference(purify_example(example)), self.tok,
                                               self.tools)
        cut = self.max_length
        p = _ids(self.tok(ex["prompt"], add_special_tokens=True)) if ex["prompt"] else []
        row = {"input_ids_chosen": (p + self._completion(ex["chosen"]))[:cut],
               "input_ids_rejected": (p + self._completion(ex["rejected"]))[:cut]}
        if "margin" in ex:
            row["margin"] = float(ex["margin"])
        return row


class GRPOPreprocessTransform(Transform):
    """Keeps the example (reward functions read its other fields) and adds the tokenised, left-truncated prompt."""

    def __call__(self, example: dict) -> dict:
        ex = purify_example(example)
        prompt = ex.get("prompt", ex.get("question", ""))
        if is_conversational(prompt):
            kw = {"tools": self.tools} if self.tools else {}
            prompt = self.tok.apply_chat_template(prompt, tokenize=False, add_generation_prompt=True, **kw)
        ids = self._prompt(prompt)
        return dict(ex, prompt=prompt, prompt_input_ids=ids, input_ids=ids, attention_mask=[1] * len(ids))


class PPOPreprocessTransform(GRPOPreprocessTransform):
    pass


class EmbeddingPreprocessTransform(Transform):
    def __init__(self, tokenizer, max_length: int | None = None, query_field: str = "query",
                 positive_field: str = "positive", negative_field: str = "negative", query_prefix: str = "",
                 passage_prefix: str = "", **kw):
        super().__init__(tokenizer, max_length=max_length, **kw)
        self.fields, self.prefix = (query_field, positive_field, negative_field), (query_prefix, passage_prefix)

    def _enc(self, text: str) -> list[int]:
        return _ids(self.tok(text, add_special_tokens=True))[: self.max_length]

    def __call__(self, example: dict) -> dict:
        q, p, n = self.fields
        row = {"query_input_ids": self._enc(self.prefix[0] + example[q]),
               "positive_input_ids": self._enc(self.prefix[1] + example[p])}
        neg = example.get(n)
        if neg:
            neg = neg[0] if isinstance(neg, (list, tuple)) else neg
            row["negative_input_ids"] = self._enc(self.prefix[1] + neg)
        return row


__all__ = ["purify_example", "is_conversational", "extract_prompt_from_preference",
           "apply_chat_template_to_preference", "Transform", "ExpandTransform", "SFTPreprocessTransform",
           "DPOPreprocessTransform", "ORPOPreprocessTransform", "CPOPreprocessTransform", "KTOPreprocessTransform",
           "BCOPreprocessTransform", "RewardPreprocessTransform", "GRPOPreprocessTransform", "PPOPreprocessTransform",
           "EmbeddingPreprocessTransform"]
