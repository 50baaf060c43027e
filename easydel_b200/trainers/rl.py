"""On-policy RL trainers: GRPO, GSPO, GFPO, RLVR, SDPO (this file) built on one rollout mixin.

Reference: easydel/trainers/group_relative_policy_optimization/_fn.py:330-812 (advantages, clipped ratio, KL to the
reference policy), group_sequence_policy_optimization (sequence-level importance ratio), group_filtered_policy_
optimization (filter completions inside each group before normalising), rlvr_trainer (verifiable rewards),
self_distillation_policy_optimization (the policy conditioned on feedback teaches itself).

A step is: host hook ``_preprocess_batch_input`` samples ``num_return_sequences`` completions per prompt (the
framework's generate loop or an eSurge engine), scores them, computes advantages and the behaviour / reference
log-probabilities without autograd; ``compute_step_loss`` then evaluates the clipped objective on micro-batches.
"""

from __future__ import annotations

import copy
import re
import typing as tp
from dataclasses import dataclass, field

import torch

from ..infra.loss_utils import LossMetrics
from ._logprob_utils import token_logprobs
from .base_trainer import Trainer
from .training_configurations import TrainingArguments, register_trainer, register_trainer_arguments
from .utils import pad_to_length


class PromptCollator:
    """Left-pads ``input_ids``; every other field is kept as a python list (answers, metadata for reward fns)."""

    def __init__(self, pad_token_id: int = 0, max_prompt_length: int | None = None):
        self.pad, self.max_len = pad_token_id, max_prompt_length

    def __call__(self, feats: list[dict]) -> dict:
        rows = [torch.as_tensor(f["input_ids"], dtype=torch.long) for f in feats]
        if self.max_len:
            rows = [r[-self.max_len:] for r in rows]
        L = max(r.shape[0] for r in rows)
        out = {"input_ids": torch.stack([pad_to_length(r, L, self.pad, left=True) for r in rows]),
               "attention_mask": torch.stack([pad_to_length(torch.ones_like(r), L, 0, left=True) for r in rows])}
        for k in feats[0]:
            if k not in ("input_ids", "attention_mask"):
                out[k] = [f[k] for f in feats]
        return out


@register_trainer_arguments("grpo")
@dataclass
class GRPOConfig(TrainingArguments):
    trainer_prefix: str | None = "grpotrainer"
    max_prompt_length: int | None = 512
    max_completion_length: int = 256
    num_return_sequences: int = 4
    beta: float = 0.04
    epsilon: float = 0.2
    epsilon_high: float | None = None
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    loss_type: str = "grpo"                  # grpo | bnpo | dr_grpo | dapo
    scale_rewards: bool = True
    importance_sampling_level: str = "token"  # token | sequence (GSPO)
    num_iterations: int = 1
    reward_weights: list[float] | None = None
    mask_truncated_completions: bool = False
    sync_ref_model: bool = False
    ref_model_mixup_alpha: float = 0.9
    ref_model_sync_steps: int = 64
    use_esurge_generation: bool = False
    skip_apply_chat_template: bool = True
    advantage_epsilon: float = 1e-4
    generation_seed: int | None = None


def first_eos_mask(completions: torch.Tensor, eos_ids: tp.Iterable[int]) -> torch.Tensor:
    """1 for every completion token up to and including the first EOS."""
    eos_ids = list(eos_ids)
    if not eos_ids:
        return torch.ones_like(completions)
    is_eos = torch.isin(completions, torch.tensor(eos_ids, device=completions.device))
    after = (is_eos.long().cumsum(1) - is_eos.long()) > 0
    return (~after).long()


def group_advantages(rewards: torch.Tensor, group: int, scale: bool = True, eps: float = 1e-4,
                     keep: torch.Tensor | None = None) -> torch.Tensor:
    """(r - mean_group) / (std_group + eps); ``keep`` restricts the statistics to retained members (GFPO)."""
    r = rewards.view(-1, group)
    if keep is None:
        mean, std = r.mean(1, keepdim=True), r.std(1, keepdim=True, unbiased=False)
        adv = r - mean
    else:
        k = keep.view(-1, group).to(r.dtype)
        n = k.sum(1, keepdim=True).clamp_min(1)
        mean = (r * k).sum(1, keepdim=True) / n
        std = (((r - mean) ** 2 * k).sum(1, keepdim=True) / n).sqrt()
        adv = (r - mean) * k
    if scale:
        adv = adv / (std + eps)
    return adv.reshape(-1)


def grpo_objective(lp, old_lp, ref_lp, adv, mask, *, epsilon=0.2, epsilon_high=None, beta=0.0, loss_type="grpo",
                   level="token", max_completion_length: int | None = None):
    """Clipped surrogate (+ k3 KL). All of ``lp, old_lp, ref_lp, mask`` are ``[N, T]``; ``adv`` is ``[N]``."""
    eh = epsilon if epsilon_high is None else epsilon_high
    log_ratio = lp - old_lp
    if level == "sequence":
        seq = (log_ratio * mask).sum(1) / mask.sum(1).clamp_min(1)
        log_ratio = seq[:, None].expand_as(lp)
    ratio = torch.exp(log_ratio)
    a = adv[:, None]
    per_tok = -torch.minimum(ratio * a, ratio.clamp(1 - epsilon, 1 + eh) * a)
    kl = None
    if beta and ref_lp is not None:
        d = ref_lp - lp
        kl = torch.exp(d) - d - 1
        per_tok = per_tok + beta * kl
    if loss_type == "grpo":
        loss = ((per_tok * mask).sum(1) / mask.sum(1).clamp_min(1)).mean()
    elif loss_type in ("bnpo", "dapo"):
        loss = (per_tok * mask).sum() / mask.sum().clamp_min(1)
    elif loss_type == "dr_grpo":
        loss = (per_tok * mask).sum() / (per_tok.shape[0] * (max_completion_length or per_tok.shape[1]))
    else:
        raise ValueError(f"unknown GRPO loss_type {loss_type!r}")
    clipped = ((ratio < 1 - epsilon) & (a < 0)) | ((ratio > 1 + eh) & (a > 0))
    stats = {"clip_ratio": (clipped.float() * mask).sum() / mask.sum().clamp_min(1)}
    if kl is not None:
        stats["kl"] = (kl.detach() * mask).sum() / mask.sum().clamp_min(1)
    return loss, stats


class RolloutMixin:
    """Sampling and scoring shared by the on-policy trainers."""

    def _setup_rollouts(self, reward_funcs, reward_processing_classes=None):
        self.reward_funcs = list(reward_funcs) if isinstance(reward_funcs, (list, tuple)) else [reward_funcs]
        self.reward_processing_classes = reward_processing_classes
        self._engine = None

    def _eos_ids(self) -> list[int]:
        e = getattr(self.processing_class, "eos_token_id", None)
        if e is None:
            e = getattr(self.model.config, "eos_token_id", None)
        if e is None:
            return []
        return list(e) if isinstance(e, (list, tuple)) else [e]

    @torch.no_grad()
    def sample_completions(self, prompt_ids: torch.Tensor, prompt_mask: torch.Tensor, n: int,
                           model=None) -> tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(completion_ids [B*n, C], completion_mask [B*n, C])``; rows of one prompt are adjacent."""
        a = self.arguments
        model = model or self.model
        ids = prompt_ids.repeat_interleave(n, 0).to(self.device)
        att = prompt_mask.repeat_interleave(n, 0).to(self.device)
        eos = self._eos_ids()
        pad = getattr(self, "pad_token_id", 0)
        if getattr(a, "use_esurge_generation", False):
            comp = self._sample_with_engine(ids, att, a)
        else:
            out = model.generate(input_ids=ids, attention_mask=att, max_new_tokens=a.max_completion_length,
                                 do_sample=True, temperature=a.temperature, top_p=a.top_p, top_k=a.top_k,
                                 eos_token_id=eos or None, pad_token_id=pad,
                                 seed=(a.generation_seed or 0) + int(self.model_state.step) * 7919)
            comp = out.sequences[:, ids.shape[1]:]
        if comp.shape[1] < a.max_completion_length:
            comp = torch.cat([comp, torch.full((comp.shape[0], a.max_completion_length - comp.shape[1]), pad,
                                               dtype=comp.dtype, device=comp.device)], 1)
        mask = first_eos_mask(comp, eos)
        if getattr(a, "mask_truncated_completions", False) and eos:
            finished = torch.isin(comp, torch.tensor(eos, device=comp.device)).any(1)
            mask = mask * finished[:, None].long()
        return comp, mask

    def _sample_with_engine(self, ids, att, a):
        from ..inference.esurge import eSurge
        from ..inference.sampling_params import SamplingParams

        if self._engine is None:
            self._engine = eSurge(self.model, tokenizer=self.processing_class,
                                  max_model_len=ids.shape[1] + a.max_completion_length,
                                  max_num_seqs=min(256, ids.shape[0]))
        prompts = [row[m.bool()].tolist() for row, m in zip(ids, att)]
        sp = SamplingParams(max_tokens=a.max_completion_length, temperature=a.temperature, top_p=a.top_p,
                            top_k=a.top_k)
        outs = self._engine.generate(prompts, sp)
        pad = getattr(self, "pad_token_id", 0)
        rows = [torch.tensor(o.outputs[0].token_ids, dtype=torch.long) for o in outs]
        return torch.stack([pad_to_length(r, a.max_completion_length, pad)[: a.max_completion_length]
                            for r in rows]).to(self.device)

    def _decode(self, ids: torch.Tensor, mask: torch.Tensor | None = None) -> list:
        tok = self.processing_class
        rows = [r[m.bool()].tolist() if m is not None else r.tolist() for r, m in
                zip(ids, mask if mask is not None else [None] * len(ids))]
        if tok is None or not hasattr(tok, "decode"):
            return rows
        return [tok.decode(r, skip_special_tokens=True) for r in rows]

    @torch.no_grad()
    def score(self, prompt_ids, prompt_mask, comp_ids, comp_mask, extras: dict, n: int) -> torch.Tensor:
        """Weighted sum of all reward functions / reward models: ``[B*n]`` and a per-function table."""
        prompts = self._decode(prompt_ids.repeat_interleave(n, 0), prompt_mask.repeat_interleave(n, 0))
        completions = self._decode(comp_ids, comp_mask)
        rep = {k: [x for x in v for _ in range(n)] for k, v in extras.items() if isinstance(v, list)}
        cols = []
        for fn in self.reward_funcs:
            if isinstance(fn, torch.nn.Module):
                ids = torch.cat([prompt_ids.repeat_interleave(n, 0).to(self.device), comp_ids], 1)
                att = torch.cat([prompt_mask.repeat_interleave(n, 0).to(self.device), comp_mask], 1)
                r = fn(input_ids=ids, attention_mask=att).logits.float()[:, 0]
            else:
                r = torch.as_tensor(fn(prompts=prompts, completions=completions, completion_ids=comp_ids,
                                       completion_mask=comp_mask, **rep), dtype=torch.float32)
            cols.append(r.to(self.device))
        table = torch.stack(cols, 1)
        w = getattr(self.arguments, "reward_weights", None)
        w = torch.ones(table.shape[1], device=self.device) if not w else torch.tensor(w, device=self.device)
        return (table * w).sum(1), table


@register_trainer("grpo")
class GRPOTrainer(RolloutMixin, Trainer):
    trainer_type = "grpo"
    arguments_class = GRPOConfig

    def __init__(self, arguments=None, model=None, reward_funcs=None, reference_model=None, processing_class=None,
                 train_dataset=None, eval_dataset=None, data_collator=None, reward_processing_classes=None, **kw):
        arguments = arguments or self.arguments_class()
        if reward_funcs is None:
            raise ValueError("`reward_funcs` is required")
        tok = processing_class if processing_class is not None else kw.pop("tokenizer", None)
        self.pad_token_id = getattr(tok, "pad_token_id", None) or 0
        self._setup_rollouts(reward_funcs, reward_processing_classes)
        super().__init__(arguments=arguments, model=model, dataset_train=kw.pop("dataset_train", train_dataset),
                         dataset_eval=kw.pop("dataset_eval", eval_dataset),
                         data_collator=data_collator or PromptCollator(self.pad_token_id, arguments.max_prompt_length),
                         processing_class=tok, **kw)
        self.reference_model = reference_model
        if self.reference_model is None and arguments.beta:
            self.reference_model = copy.deepcopy(self.model).eval().requires_grad_(False)
        for fn in self.reward_funcs:
            if isinstance(fn, torch.nn.Module):
                fn.eval().requires_grad_(False)

    # rollout-side hooks that the variants override ------------------------------------------------
    def _advantages(self, rewards, comp_mask, n) -> tuple[torch.Tensor, dict]:
        a = self.arguments
        return group_advantages(rewards, n, a.scale_rewards, a.advantage_epsilon), {}

    def _preprocess_batch_input(self, state, batch, is_train):
        a = self.arguments
        n = a.num_return_sequences
        p_ids, p_mask = batch["input_ids"], batch["attention_mask"]
        extras = {k: v for k, v in batch.items() if k not in ("input_ids", "attention_mask")}
        comp, cmask = self.sample_completions(p_ids, p_mask, n)
        rewards, table = self.score(p_ids, p_mask, comp, cmask, extras, n)
        adv, extra_metrics = self._advantages(rewards, cmask, n)
        ids = torch.cat([p_ids.repeat_interleave(n, 0).to(self.device), comp], 1)
        att = torch.cat([p_mask.repeat_interleave(n, 0).to(self.device), cmask], 1)
        lmask = torch.cat([torch.zeros_like(p_mask.repeat_interleave(n, 0)).to(self.device), cmask], 1)
        new = {"input_ids": ids, "attention_mask": att, "loss_mask": lmask, "advantages": adv}
        with torch.no_grad():
            was = self.model.training
            self.model.eval()
            new["old_logps"] = self._chunked_logps(self.model, ids, att, lmask)
            if self.reference_model is not None and a.beta:
                new["ref_logps"] = self._chunked_logps(self.reference_model, ids, att, lmask)
            self.model.train(was)
        new.update(self._extra_rollout_tensors(batch, new, comp, cmask, rewards, n))
        metrics = {"rewards/mean": float(rewards.mean()), "rewards/std": float(rewards.std(unbiased=False)),
                   "completions/mean_length": float(cmask.sum(1).float().mean())}
        for i in range(table.shape[1]):
            name = getattr(self.reward_funcs[i], "__name__", type(self.reward_funcs[i]).__name__)
            metrics[f"rewards/{name}"] = float(table[:, i].mean())
        metrics.update(extra_metrics)
        return new, metrics

    def _extra_rollout_tensors(self, batch, new, comp, cmask, rewards, n) -> dict:
        return {}

    def _chunked_logps(self, model, ids, att, lmask):
        bs = max(1, self.micro_batch_size * self.arguments.num_return_sequences)
        outs = []
        for s in range(0, ids.shape[0], bs):
            lp, _, _, _ = token_logprobs(model, ids[s:s + bs], att[s:s + bs], lmask[s:s + bs],
                                         temperature=self.arguments.temperature)
            outs.append(lp.detach())
        return torch.cat(outs, 0)

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        lp, m, _, out = token_logprobs(model, batch["input_ids"], batch["attention_mask"], batch["loss_mask"],
                                       temperature=a.temperature)
        loss, stats = grpo_objective(lp, batch["old_logps"], batch.get("ref_logps"), batch["advantages"], m,
                                     epsilon=a.epsilon, epsilon_high=a.epsilon_high, beta=a.beta,
                                     loss_type=a.loss_type, level=a.importance_sampling_level,
                                     max_completion_length=a.max_completion_length)
        return LossMetrics(loss=loss * loss_scale, other_metrics=stats)


# ----------------------------------------------------------------------------------------- GSPO
@register_trainer_arguments("gspo")
@dataclass
class GSPOConfig(GRPOConfig):
    trainer_prefix: str | None = "gspotrainer"
    importance_sampling_level: str = "sequence"
    epsilon: float = 3e-4
    epsilon_high: float | None = 4e-4
    beta: float = 0.0
    loss_type: str = "grpo"


@register_trainer("gspo")
class GSPOTrainer(GRPOTrainer):
    """Sequence-level importance ratios with tight clipping (easydel/trainers/group_sequence_policy_optimization)."""

    trainer_type = "gspo"
    arguments_class = GSPOConfig


# ----------------------------------------------------------------------------------------- GFPO
@register_trainer_arguments("gfpo")
@dataclass
class GFPOConfig(GRPOConfig):
    trainer_prefix: str | None = "gfpotrainer"
    gfpo_group_size: int | None = None       # sample this many, ...
    gfpo_retain_count: int = 2               # ... keep the best `retain` per group
    gfpo_metric: str = "length"              # length | token_efficiency
    gfpo_adaptive: bool = False              # harder prompts (lower mean reward) retain more


@register_trainer("gfpo")
class GFPOTrainer(GRPOTrainer):
    """Group-filtered policy optimisation: rank the completions of each group by a secondary metric (short length,
    reward per token), keep the top ``retain`` and normalise advantages over the survivors only."""

    trainer_type = "gfpo"
    arguments_class = GFPOConfig

    def _advantages(self, rewards, comp_mask, n):
        a = self.arguments
        lengths = comp_mask.sum(1).float().clamp_min(1)
        metric = -lengths if a.gfpo_metric == "length" else rewards / lengths
        r, m = rewards.view(-1, n), metric.view(-1, n)
        retain = torch.full((r.shape[0],), min(a.gfpo_retain_count, n), device=r.device)
        if a.gfpo_adaptive:
            hardness = 1 - (r.mean(1) - r.mean()) .sigmoid()
            retain = (retain.float() * (0.5 + hardness)).round().clamp(1, n).long()
        order = m.argsort(1, descending=True)
        rank = torch.empty_like(order)
        rank.scatter_(1, order, torch.arange(n, device=r.device)[None].expand_as(order))
        keep = (rank < retain[:, None]).reshape(-1)
        adv = group_advantages(rewards, n, a.scale_rewards, a.advantage_epsilon, keep=keep)
        return adv, {"gfpo/retained_fraction": float(keep.float().mean())}


# ----------------------------------------------------------------------------------------- RLVR
_BOXED = re.compile(r"\\boxed\{([^{}]*)\}")
_HASHES = re.compile(r"####\s*([^\n]+)")
_NUMBER = re.compile(r"-?\d+(?:[\.,]\d+)*(?:/\d+)?")


def extract_final_answer(text: str) -> str | None:
    """``\\boxed{..}`` first, then ``#### ..`` (GSM8K style), then the last number in the text."""
    if not isinstance(text, str):
        return None
    m = _BOXED.findall(text)
    if m:
        return m[-1].strip()
    m = _HASHES.findall(text)
    if m:
        return m[-1].strip()
    m = _NUMBER.findall(text)
    return m[-1] if m else None


def _normalise_answer(s: str | None) -> str | None:
    if s is None:
        return None
    s = str(s).strip().replace(",", "").replace("$", "").rstrip(".").lower()
    try:
        if "/" in s:
            a, b = s.split("/")
            return repr(float(a) / float(b))
        return repr(float(s))
    except ValueError:
        return s


class MathVerifier:
    """1.0 when the extracted final answer equals the row's ``answer`` (numerically when both parse)."""

    __name__ = "math_verifier"

    def __init__(self, answer_key: str = "answer", correct: float = 1.0, wrong: float = 0.0):
        self.key, self.correct, self.wrong = answer_key, correct, wrong

    def __call__(self, prompts, completions, **kw):
        answers = kw.get(self.key)
        if answers is None:
            raise KeyError(f"dataset rows need an '{self.key}' field for MathVerifier")
        return [self.correct if _normalise_answer(extract_final_answer(c)) == _normalise_answer(
            extract_final_answer(a) if isinstance(a, str) and ("####" in a or "\\boxed" in a) else a) else self.wrong
            for c, a in zip(completions, answers)]


class FormatVerifier:
    """Reward for matching a regular expression (e.g. ``<think>..</think><answer>..</answer>``)."""

    __name__ = "format_verifier"

    def __init__(self, pattern: str = r"^<think>.*?</think>\s*<answer>.*?</answer>\s*$", reward: float = 0.5):
        self.rx, self.reward = re.compile(pattern, re.S), reward

    def __call__(self, prompts, completions, **kw):
        return [self.reward if isinstance(c, str) and self.rx.match(c) else 0.0 for c in completions]


class LengthPenaltyVerifier:
    """Linear penalty once a completion exceeds ``target`` tokens."""

    __name__ = "length_penalty"

    def __init__(self, target: int, weight: float = 0.001):
        self.target, self.weight = target, weight

    def __call__(self, prompts, completions, completion_mask=None, **kw):
        n = completion_mask.sum(1).tolist() if completion_mask is not None else [len(c) for c in completions]
        return [-self.weight * max(0, x - self.target) for x in n]


class CodeExecutionVerifier:
    """Runs the completion's python code block against the row's ``tests`` in a subprocess with a time limit."""

    __name__ = "code_verifier"

    def __init__(self, tests_key: str = "tests", timeout: float = 5.0):
        self.key, self.timeout = tests_key, timeout

    def __call__(self, prompts, completions, **kw):
        import subprocess
        import sys
        import tempfile

        out = []
        for c, t in zip(completions, kw.get(self.key) or [""] * len(completions)):
            m = re.findall(r"```(?:python)?\n(.*?)```", c if isinstance(c, str) else "", re.S)
            code = (m[-1] if m else (c if isinstance(c, str) else "")) + "\n" + (t or "")
            with tempfile.NamedTemporaryFile("w", suffix=".py", delete=True) as f:
                f.write(code)
                f.flush()
                try:
                    r = subprocess.run([sys.executable, f.name], capture_output=True, timeout=self.timeout)
                    out.append(1.0 if r.returncode == 0 else 0.0)
                except subprocess.TimeoutExpired:
                    out.append(0.0)
        return out


@register_trainer_arguments("rlvr")
@dataclass
class RLVRConfig(GRPOConfig):
    trainer_prefix: str | None = "rlvrtrainer"
    answer_key: str = "answer"
    format_pattern: str | None = None
    format_reward: float = 0.0
    length_penalty_target: int | None = None
    length_penalty_weight: float = 0.001
    beta: float = 0.0


@register_trainer("rlvr")
class RLVRTrainer(GRPOTrainer):
    """GRPO whose rewards are programmatic verifiers (easydel/trainers/rlvr_trainer). Without explicit
    ``reward_funcs`` a :class:`MathVerifier` on ``answer_key`` (+ optional format / length terms) is used."""

    trainer_type = "rlvr"
    arguments_class = RLVRConfig

    def __init__(self, arguments=None, model=None, reward_funcs=None, verifiers=None, **kw):
        arguments = arguments or RLVRConfig()
        fns = list(verifiers or reward_funcs or [])
        if not fns:
            fns = [MathVerifier(arguments.answer_key)]
            if arguments.format_pattern and arguments.format_reward:
                fns.append(FormatVerifier(arguments.format_pattern, arguments.format_reward))
            if arguments.length_penalty_target:
                fns.append(LengthPenaltyVerifier(arguments.length_penalty_target, arguments.length_penalty_weight))
        super().__init__(arguments=arguments, model=model, reward_funcs=fns, **kw)


# ----------------------------------------------------------------------------------------- SDPO
@register_trainer_arguments("sdpo")
@dataclass
class SDPOConfig(GRPOConfig):
    trainer_prefix: str | None = "SDPO"
    max_feedback_length: int = 256
    distillation_type: str = "jsd"           # jsd | kl
    beta: float = 0.0
    success_threshold: float = 0.5           # without a feedback function: rollouts scoring above it teach the others


def sdpo_token_loss(student_lp: torch.Tensor, teacher_lp: torch.Tensor, kind: str = "jsd") -> torch.Tensor:
    """Sampled-token estimate of the divergence between the student and its feedback-conditioned self."""
    if kind == "kl":
        return student_lp - teacher_lp
    if kind == "jsd":
        mix = torch.logaddexp(student_lp, teacher_lp) - torch.log(torch.tensor(2.0))
        return student_lp - mix
    raise ValueError(f"unknown distillation_type {kind!r}")


@register_trainer("sdpo")
class SDPOTrainer(GRPOTrainer):
    """Self-distillation policy optimisation: the current policy, shown its own attempt plus feedback, scores the
    attempt's tokens; the gap between that self-teacher and the plain policy is the per-token learning signal
    (easydel/trainers/self_distillation_policy_optimization). ``feedback_func(prompts, completions, rewards, **row)``
    returns one feedback string (or token list) per completion; without it, the best successful completion of the
    same group serves as feedback for the others."""

    trainer_type = "sdpo"
    arguments_class = SDPOConfig

    def __init__(self, *a, feedback_func=None, **kw):
        self.feedback_func = feedback_func
        super().__init__(*a, **kw)

    def _feedback_ids(self, batch, comp, cmask, rewards, n) -> list[list[int]]:
        a = self.arguments
        tok = self.processing_class
        N = comp.shape[0]
        if self.feedback_func is not None:
            prompts = self._decode(batch["input_ids"].repeat_interleave(n, 0),
                                   batch["attention_mask"].repeat_interleave(n, 0))
            fb = self.feedback_func(prompts=prompts, completions=self._decode(comp, cmask), rewards=rewards.tolist())
            rows = [tok(f, add_special_tokens=False)["input_ids"] if isinstance(f, str) else list(f) for f in fb]
        else:
            rows = []
            r = rewards.view(-1, n)
            best = r.argmax(1)
            for i in range(N):
                g, j = divmod(i, n)
                b = g * n + int(best[g])
                if float(r[g, best[g]]) > a.success_threshold and b != i:
                    rows.append(comp[b][cmask[b].bool()].tolist())
                else:
                    rows.append([])
        return [r[: a.max_feedback_length] for r in rows]

    def _extra_rollout_tensors(self, batch, new, comp, cmask, rewards, n):
        a = self.arguments
        fb = self._feedback_ids(batch, comp, cmask, rewards, n)
        F_len = max(1, max(len(r) for r in fb))
        pad = self.pad_token_id
        fb_ids = torch.tensor([[pad] * (F_len - len(r)) + r for r in fb], dtype=torch.long, device=self.device)
        fb_mask = torch.tensor([[0] * (F_len - len(r)) + [1] * len(r) for r in fb], dtype=torch.long,
                               device=self.device)
        p_ids = batch["input_ids"].repeat_interleave(n, 0).to(self.device)
        p_mask = batch["attention_mask"].repeat_interleave(n, 0).to(self.device)
        t_ids = torch.cat([p_ids, fb_ids, comp], 1)
        t_att = torch.cat([p_mask, fb_mask, cmask], 1)
        t_lm = torch.cat([torch.zeros_like(p_mask), torch.zeros_like(fb_mask), cmask], 1)
        with torch.no_grad():
            was = self.model.training
            self.model.eval()
            t_lp = self._chunked_logps(self.model, t_ids, t_att, t_lm)
            self.model.train(was)
        C = comp.shape[1]
        teacher = torch.zeros_like(new["old_logps"])
        teacher[:, -C:] = t_lp[:, -C:]
        has_fb = torch.tensor([len(r) > 0 for r in fb], device=self.device)
        return {"teacher_logps": teacher, "has_feedback": has_fb}

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        lp, m, _, _ = token_logprobs(model, batch["input_ids"], batch["attention_mask"], batch["loss_mask"],
                                     temperature=a.temperature)
        m = m * batch["has_feedback"][:, None].to(m.dtype)
        # per-token advantage log(teacher / student) weights the score function; its gradient is that of the
        # sampled-token divergence estimate below
        per_tok = sdpo_token_loss(lp, batch["teacher_logps"], a.distillation_type)
        adv = (batch["teacher_logps"] - lp).detach()
        loss = (per_tok * m).sum() / m.sum().clamp_min(1)
        stats = {"sdpo/advantage": (adv * m).sum() / m.sum().clamp_min(1)}
        if a.beta and "ref_logps" in batch:
            d = batch["ref_logps"] - lp
            kl = torch.exp(d) - d - 1
            loss = loss + a.beta * (kl * m).sum() / m.sum().clamp_min(1)
        return LossMetrics(loss=loss * loss_scale, other_metrics=stats)
