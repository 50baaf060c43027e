"""Knowledge-distillation trainers: logit distillation, GKD, sequence-level KD, sparse (top-k) distillation and
on-policy distillation.

Reference: easydel/trainers/distillation_trainer (KL to teacher logits mixed with the hard-label loss, optional
hidden-state / attention matching), generalized_knowledge_distillation_trainer (generalised JSD with on-policy
student samples), seq_kd_trainer (train on teacher generations), sparse_distillation_trainer (teacher top-k
logits only), on_policy_distillation_trainer (reverse KL on student samples).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as tF

from ..infra.loss_utils import LossMetrics
from .base_trainer import Trainer
from .rl import PromptCollator, RolloutMixin
from .training_configurations import TrainingArguments, register_trainer, register_trainer_arguments


def _masked_token_mean(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return (x * mask).sum() / mask.sum().clamp_min(1)


def distillation_kl(student_logits, teacher_logits, mask, temperature: float = 1.0, reverse: bool = False):
    """Token-mean KL(teacher || student) (or the reverse), scaled by T^2 as usual."""
    s = torch.log_softmax(student_logits.float() / temperature, -1)
    t = torch.log_softmax(teacher_logits.float() / temperature, -1)
    kl = (s.exp() * (s - t)).sum(-1) if reverse else (t.exp() * (t - s)).sum(-1)
    return _masked_token_mean(kl, mask) * temperature ** 2


def generalized_jsd(student_logits, teacher_logits, mask, beta: float = 0.5, temperature: float = 1.0):
    """Generalised Jensen-Shannon divergence of GKD: ``beta = 0`` is forward KL, ``beta = 1`` reverse KL."""
    s = torch.log_softmax(student_logits.float() / temperature, -1)
    t = torch.log_softmax(teacher_logits.float() / temperature, -1)
    if beta <= 0:
        d = (t.exp() * (t - s)).sum(-1)
    elif beta >= 1:
        d = (s.exp() * (s - t)).sum(-1)
    else:
        mix = torch.logsumexp(torch.stack([s + math.log(1 - beta), t + math.log(beta)]), 0)
        d = beta * (t.exp() * (t - mix)).sum(-1) + (1 - beta) * (s.exp() * (s - mix)).sum(-1)
    return _masked_token_mean(d, mask)


def sparse_topk_kl(student_logits, teacher_logits, mask, k: int = 32, temperature: float = 1.0,
                   renormalise: bool = True):
    """KL restricted to the teacher's top-k tokens (the teacher's mass elsewhere is dropped or kept as a tail bin)."""
    t = teacher_logits.float() / temperature
    s = torch.log_softmax(student_logits.float() / temperature, -1)
    tv, ti = t.topk(k, -1)
    if renormalise:
        tl = torch.log_softmax(tv, -1)
        sl = torch.log_softmax(s.gather(-1, ti), -1)
        kl = (tl.exp() * (tl - sl)).sum(-1)
    else:
        tl_full = torch.log_softmax(t, -1)
        tl = tl_full.gather(-1, ti)
        sl = s.gather(-1, ti)
        tail_t = torch.log1p(-tl.exp().sum(-1).clamp_max(1 - 1e-6))
        tail_s = torch.log1p(-sl.exp().sum(-1).clamp_max(1 - 1e-6))
        kl = (tl.exp() * (tl - sl)).sum(-1) + tail_t.exp() * (tail_t - tail_s)
    return _masked_token_mean(kl, mask) * temperature ** 2


@register_trainer_arguments("distillation")
@dataclass
class DistillationConfig(TrainingArguments):
    trainer_prefix: str | None = "distillationtrainer"
    temperature: float = 2.0
    alpha: float = 0.9                        # weight of the distillation term vs. the hard-label loss
    hidden_state_loss_weight: float = 0.0
    hidden_state_layers: tuple[int, ...] | None = None
    reverse_kl: bool = False


class _TeacherMixin:
    def _setup_teacher(self, teacher_model):
        if teacher_model is None:
            raise ValueError("`teacher_model` is required")
        self.teacher_model = teacher_model.eval().requires_grad_(False)

    @staticmethod
    def _shift(batch):
        labels = batch.get("labels", batch["input_ids"])
        att = batch.get("attention_mask")
        mask = (labels[:, 1:] != -100)
        if att is not None:
            mask = mask & att[:, 1:].bool()
        return labels, mask.float()


@register_trainer("distillation")
class DistillationTrainer(_TeacherMixin, Trainer):
    trainer_type = "distillation"
    arguments_class = DistillationConfig

    def __init__(self, arguments=None, student_model=None, teacher_model=None, model=None, **kw):
        arguments = arguments or self.arguments_class()
        self._setup_teacher(teacher_model)
        kw.setdefault("dataset_train", kw.pop("train_dataset", None))
        kw.setdefault("dataset_eval", kw.pop("eval_dataset", None))
        super().__init__(arguments=arguments, model=student_model if student_model is not None else model, **kw)

    def _divergence(self, s_logits, t_logits, mask):
        a = self.arguments
        return distillation_kl(s_logits, t_logits, mask, a.temperature, a.reverse_kl)

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        labels, mask = self._shift(batch)
        call = {k: v for k, v in batch.items() if k in ("input_ids", "attention_mask", "segment_ids", "position_ids")}
        want_h = a.hidden_state_loss_weight > 0
        out = model(**call, output_hidden_states=want_h)
        with torch.no_grad():
            t_out = self.teacher_model(**call, output_hidden_states=want_h)
        s_logits, t_logits = out.logits[:, :-1], t_out.logits[:, :-1]
        V = min(s_logits.shape[-1], t_logits.shape[-1])
        kd = self._divergence(s_logits[..., :V], t_logits[..., :V], mask)
        tgt = labels[:, 1:].masked_fill(mask == 0, -100)
        ce = tF.cross_entropy(s_logits.float().reshape(-1, s_logits.shape[-1]), tgt.reshape(-1), ignore_index=-100)
        loss = a.alpha * kd + (1 - a.alpha) * ce
        stats = {"distill/kd_loss": kd.detach(), "distill/ce_loss": ce.detach()}
        if want_h:
            layers = a.hidden_state_layers or (-1,)
            hs = sum(tF.mse_loss(out.hidden_states[i].float(), t_out.hidden_states[i].float()) for i in layers)
            loss = loss + a.hidden_state_loss_weight * hs
            stats["distill/hidden_loss"] = hs.detach()
        return LossMetrics(loss=loss * loss_scale, other_metrics=stats)


@register_trainer_arguments("sparse_distillation")
@dataclass
class SparseDistillationConfig(DistillationConfig):
    trainer_prefix: str | None = "sparsedistillationtrainer"
    top_k: int = 32
    renormalise_topk: bool = True


@register_trainer("sparse_distillation")
class SparseDistillationTrainer(DistillationTrainer):
    """Matches only the teacher's top-k logits; rows may also carry precomputed ``teacher_topk_logits`` /
    ``teacher_topk_indices`` so that no teacher forward is needed."""

    trainer_type = "sparse_distillation"
    arguments_class = SparseDistillationConfig

    def _divergence(self, s_logits, t_logits, mask):
        a = self.arguments
        return sparse_topk_kl(s_logits, t_logits, mask, a.top_k, a.temperature, a.renormalise_topk)


@register_trainer_arguments("seq_kd")
@dataclass
class SeqKDConfig(TrainingArguments):
    trainer_prefix: str | None = "seqkdtrainer"
    max_prompt_length: int | None = 512
    max_completion_length: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    num_return_sequences: int = 1


@register_trainer("seq_kd")
class SeqKDTrainer(_TeacherMixin, RolloutMixin, Trainer):
    """Sequence-level KD: the teacher generates a completion for each prompt and the student is trained on it
    with the ordinary next-token loss (easydel/trainers/seq_kd_trainer)."""

    trainer_type = "seq_kd"
    arguments_class = SeqKDConfig

    def __init__(self, arguments=None, model=None, teacher_model=None, processing_class=None, train_dataset=None,
                 eval_dataset=None, data_collator=None, **kw):
        arguments = arguments or SeqKDConfig()
        self._setup_teacher(teacher_model)
        self._setup_rollouts([])
        self.pad_token_id = getattr(processing_class, "pad_token_id", None) or 0
        super().__init__(arguments=arguments, model=model, dataset_train=kw.pop("dataset_train", train_dataset),
                         dataset_eval=kw.pop("dataset_eval", eval_dataset),
                         data_collator=data_collator or PromptCollator(self.pad_token_id, arguments.max_prompt_length),
                         processing_class=processing_class, **kw)

    def _preprocess_batch_input(self, state, batch, is_train):
        p, pm = batch["input_ids"], batch["attention_mask"]
        comp, cm = self.sample_completions(p, pm, 1, model=self.teacher_model)
        ids = torch.cat([p.to(self.device), comp], 1)
        att = torch.cat([pm.to(self.device), cm], 1)
        labels = torch.cat([torch.full_like(p, -100).to(self.device), comp.masked_fill(cm == 0, -100)], 1)
        return {"input_ids": ids, "attention_mask": att, "labels": labels}, {}


@register_trainer_arguments("gkd")
@dataclass
class GKDConfig(SeqKDConfig):
    trainer_prefix: str | None = "gkdtrainer"
    lmbda: float = 0.5        # probability that a step trains on student-generated completions
    beta: float = 0.5         # interpolation of the generalised JSD
    seq_kd: bool = False      # off-policy steps use teacher generations instead of dataset completions
    disable_dropout: bool = True


@register_trainer("gkd")
class GKDTrainer(SeqKDTrainer):
    """Generalised knowledge distillation: with probability ``lmbda`` the completion is sampled from the student
    (on-policy); the loss is the generalised JSD between teacher and student token distributions."""

    trainer_type = "gkd"
    arguments_class = GKDConfig

    def _preprocess_batch_input(self, state, batch, is_train):
        a = self.arguments
        g = torch.Generator().manual_seed(1000003 * int(state.step) + 11)
        on_policy = bool(torch.rand((), generator=g) < a.lmbda)
        p, pm = batch["input_ids"], batch["attention_mask"]
        if not on_policy and "completion_input_ids" in batch and not a.seq_kd:
            rows = [torch.as_tensor(r, dtype=torch.long) for r in batch["completion_input_ids"]]
            L = max(len(r) for r in rows)
            comp = torch.stack([torch.cat([r, torch.full((L - len(r),), self.pad_token_id)]) for r in rows])
            cm = torch.stack([torch.cat([torch.ones(len(r)), torch.zeros(L - len(r))]) for r in rows]).long()
            comp, cm = comp.to(self.device), cm.to(self.device)
        else:
            comp, cm = self.sample_completions(p, pm, 1, model=self.model if on_policy else self.teacher_model)
        ids = torch.cat([p.to(self.device), comp], 1)
        att = torch.cat([pm.to(self.device), cm], 1)
        lm = torch.cat([torch.zeros_like(pm).to(self.device), cm], 1)
        return {"input_ids": ids, "attention_mask": att, "loss_mask": lm}, {"gkd/on_policy": float(on_policy)}

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        call = {"input_ids": batch["input_ids"], "attention_mask": batch["attention_mask"]}
        s = model(**call).logits[:, :-1]
        with torch.no_grad():
            t = self.teacher_model(**call).logits[:, :-1]
        V = min(s.shape[-1], t.shape[-1])
        mask = batch["loss_mask"][:, 1:].float()
        loss = generalized_jsd(s[..., :V], t[..., :V], mask, a.beta, a.temperature)
        return LossMetrics(loss=loss * loss_scale, other_metrics={"gkd/jsd": loss.detach()})


@register_trainer_arguments("on_policy_distillation")
@dataclass
class OnPolicyDistillationConfig(SeqKDConfig):
    trainer_prefix: str | None = "onpolicydistillationtrainer"
    kl_mode: str = "reverse"      # reverse (mode seeking, default) | forward | sampled
    disable_dropout: bool = True


@register_trainer("on_policy_distillation")
class OnPolicyDistillationTrainer(SeqKDTrainer):
    """Always samples from the student and minimises the reverse KL to the teacher on those samples. ``sampled``
    uses only the sampled token (``log pi_s - log pi_t`` as a per-token reward), which needs no full-vocabulary
    teacher logits."""

    trainer_type = "on_policy_distillation"
    arguments_class = OnPolicyDistillationConfig

    def _preprocess_batch_input(self, state, batch, is_train):
        p, pm = batch["input_ids"], batch["attention_mask"]
        comp, cm = self.sample_completions(p, pm, 1, model=self.model)
        ids = torch.cat([p.to(self.device), comp], 1)
        att = torch.cat([pm.to(self.device), cm], 1)
        lm = torch.cat([torch.zeros_like(pm).to(self.device), cm], 1)
        new = {"input_ids": ids, "attention_mask": att, "loss_mask": lm}
        if self.arguments.kl_mode == "sampled":
            from ._logprob_utils import token_logprobs

            with torch.no_grad():
                new["teacher_logps"] = token_logprobs(self.teacher_model, ids, att, lm)[0]
        return new, {}

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        mask = batch["loss_mask"][:, 1:].float()
        if a.kl_mode == "sampled":
            from ._logprob_utils import token_logprobs

            lp = token_logprobs(model, batch["input_ids"], batch["attention_mask"], batch["loss_mask"])[0]
            adv = (batch["teacher_logps"] - lp).detach()            # reward: how much the teacher likes the token
            loss = -_masked_token_mean(adv * lp, mask)
            return LossMetrics(loss=loss * loss_scale,
                               other_metrics={"opd/reverse_kl_estimate": -_masked_token_mean(adv, mask)})
        call = {"input_ids": batch["input_ids"], "attention_mask": batch["attention_mask"]}
        s = model(**call).logits[:, :-1]
        with torch.no_grad():
            t = self.teacher_model(**call).logits[:, :-1]
        V = min(s.shape[-1], t.shape[-1])
        loss = distillation_kl(s[..., :V], t[..., :V], mask, 1.0, reverse=a.kl_mode == "reverse")
        return LossMetrics(loss=loss * loss_scale, other_metrics={"opd/kl": loss.detach()})
