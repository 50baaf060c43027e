"""Preference-optimisation trainers: DPO (14 loss variants), ORPO, CPO/SimPO, KTO, BCO.

Reference: easydel/trainers/direct_preference_optimization_trainer/_fn.py:445-1213 (losses, concatenated forward,
training step), odds_ratio_preference_optimization_trainer, contrastive_preference_optimization_trainer,
kto_trainer, binary_classifier_optimization_trainer.

Batch layout (same field names as the reference's collators): ``prompt_input_ids``, ``prompt_attention_mask``,
``chosen_input_ids``, ``chosen_attention_mask``, ``rejected_input_ids``, ``rejected_attention_mask`` and, when
reference log-probabilities were precomputed, ``reference_chosen_logps`` / ``reference_rejected_logps``.
Chosen and rejected rows run through the policy in one concatenated batch; the reference model (a frozen copy
or a separate model) runs without autograd.
"""

from __future__ import annotations

import copy
import typing as tp
from dataclasses import dataclass

import torch
import torch.nn.functional as tF

from ..infra.loss_utils import LossMetrics
from ._logprob_utils import sequence_logprobs
from .base_trainer import Trainer
from .training_configurations import TrainingArguments, register_trainer, register_trainer_arguments
from .utils import pad_to_length

LOSS_TYPES = ("sigmoid", "hinge", "ipo", "exo_pair", "nca_pair", "robust", "bco_pair", "sppo_hard", "aot",
              "aot_pair", "apo_zero", "apo_down", "discopop", "kto")


def dpo_loss(policy_chosen: torch.Tensor, policy_rejected: torch.Tensor, ref_chosen: torch.Tensor,
             ref_rejected: torch.Tensor, *, beta: float = 0.1, label_smoothing: float = 0.0,
             loss_type: str = "sigmoid", reference_free: bool = False, discopop_tau: float = 0.05,
             running_delta: torch.Tensor | float = 0.0):
    """Returns ``(losses [B or 2B], chosen_rewards [B], rejected_rewards [B])`` for one of the 14 variants."""
    if reference_free:
        ref_chosen, ref_rejected = torch.zeros_like(ref_chosen), torch.zeros_like(ref_rejected)
    pi_logratios = policy_chosen - policy_rejected
    ref_logratios = ref_chosen - ref_rejected
    logits = pi_logratios - ref_logratios
    c_lr = policy_chosen - ref_chosen
    r_lr = policy_rejected - ref_rejected
    ls = label_smoothing
    if loss_type == "sigmoid":
        losses = -tF.logsigmoid(beta * logits) * (1 - ls) - tF.logsigmoid(-beta * logits) * ls
    elif loss_type == "robust":
        losses = (-tF.logsigmoid(beta * logits) * (1 - ls) + tF.logsigmoid(-beta * logits) * ls) / (1 - 2 * ls)
    elif loss_type == "exo_pair":
        eps = ls if ls > 0 else 1e-3
        p = torch.sigmoid(beta * logits)
        losses = p * (tF.logsigmoid(beta * logits) - torch.log(torch.tensor(1 - eps))) + \
            (1 - p) * (tF.logsigmoid(-beta * logits) - torch.log(torch.tensor(eps)))
    elif loss_type == "hinge":
        losses = torch.relu(1 - beta * logits)
    elif loss_type == "ipo":
        losses = (logits - 1 / (2 * beta)) ** 2
    elif loss_type == "bco_pair":
        losses = -tF.logsigmoid(beta * c_lr - running_delta) - tF.logsigmoid(-(beta * r_lr - running_delta))
    elif loss_type == "sppo_hard":
        losses = (c_lr - 0.5 / beta) ** 2 + (r_lr + 0.5 / beta) ** 2
    elif loss_type == "nca_pair":
        losses = -tF.logsigmoid(beta * c_lr) - 0.5 * tF.logsigmoid(-beta * c_lr) - 0.5 * tF.logsigmoid(-beta * r_lr)
    elif loss_type == "aot_pair":
        delta = torch.sort(c_lr, dim=0).values - torch.sort(r_lr, dim=0).values
        losses = -tF.logsigmoid(beta * delta) * (1 - ls) - tF.logsigmoid(-beta * delta) * ls
    elif loss_type == "aot":
        delta = torch.sort(pi_logratios, dim=0).values - torch.sort(ref_logratios, dim=0).values
        losses = -tF.logsigmoid(beta * delta) * (1 - ls) - tF.logsigmoid(-beta * delta) * ls
    elif loss_type == "apo_zero":
        losses = (1 - torch.sigmoid(beta * c_lr)) + torch.sigmoid(beta * r_lr)
    elif loss_type == "apo_down":
        losses = torch.sigmoid(beta * c_lr) + (1 - torch.sigmoid(beta * (c_lr - r_lr)))
    elif loss_type == "discopop":
        lg = beta * logits
        mod = torch.sigmoid(lg / discopop_tau)
        losses = -tF.logsigmoid(lg) * (1 - mod) + torch.exp(-lg) * mod
    elif loss_type == "kto":
        chosen_kl = c_lr.mean().clamp_min(0)
        rejected_kl = r_lr.mean().clamp_min(0)
        losses = torch.cat([1 - torch.sigmoid(beta * (c_lr - rejected_kl)),
                            1 - torch.sigmoid(beta * (chosen_kl - r_lr))], 0)
    else:
        raise ValueError(f"unknown DPO loss_type {loss_type!r}; choose from {LOSS_TYPES}")
    return losses, (beta * c_lr).detach(), (beta * r_lr).detach()


def concatenated_inputs(batch: dict, pad_token_id: int = 0) -> dict:
    """[prompt ; chosen] and [prompt ; rejected] stacked along the batch axis, right-padded to one length."""
    p, pm = batch["prompt_input_ids"], batch["prompt_attention_mask"]
    c, cm = batch["chosen_input_ids"], batch["chosen_attention_mask"]
    r, rm = batch["rejected_input_ids"], batch["rejected_attention_mask"]
    L = max(c.shape[1], r.shape[1])

    def padr(t, v):
        if t.shape[1] == L:
            return t
        return torch.cat([t, torch.full((t.shape[0], L - t.shape[1]), v, dtype=t.dtype, device=t.device)], 1)

    comp = torch.cat([padr(c, pad_token_id), padr(r, pad_token_id)], 0)
    comp_m = torch.cat([padr(cm, 0), padr(rm, 0)], 0)
    ids = torch.cat([torch.cat([p, p], 0), comp], 1)
    att = torch.cat([torch.cat([pm, pm], 0), comp_m], 1)
    loss_mask = torch.cat([torch.zeros_like(torch.cat([pm, pm], 0)), comp_m], 1)
    return {"input_ids": ids, "attention_mask": att, "loss_mask": loss_mask}


def concatenated_forward(model, batch: dict, *, average: bool = False, pad_token_id: int = 0, want_nll: bool = False):
    cat = concatenated_inputs(batch, pad_token_id)
    logps, ntok, out = sequence_logprobs(model, cat["input_ids"], cat["attention_mask"], cat["loss_mask"])
    B = batch["chosen_input_ids"].shape[0]
    res = {"chosen_logps": logps[:B], "rejected_logps": logps[B:], "chosen_tokens": ntok[:B],
           "rejected_tokens": ntok[B:], "aux_loss": getattr(out, "aux_loss", None)}
    if average:
        res["chosen_avg"] = logps[:B] / ntok[:B].clamp_min(1)
        res["rejected_avg"] = logps[B:] / ntok[B:].clamp_min(1)
    if want_nll:
        res["nll"] = -(logps[:B].sum() / ntok[:B].sum().clamp_min(1))
    return res


class DPODataCollator:
    """Pads prompts on the left and completions on the right (easydel/trainers/utils.py DPO collator)."""

    def __init__(self, pad_token_id: int = 0, max_prompt_length: int | None = None,
                 max_completion_length: int | None = None):
        self.pad, self.mp, self.mc = pad_token_id, max_prompt_length, max_completion_length

    def __call__(self, feats: list[dict]) -> dict:
        out = {}
        for key, left, cap in (("prompt", True, self.mp), ("chosen", False, self.mc), ("rejected", False, self.mc)):
            rows = [torch.as_tensor(f[f"{key}_input_ids"], dtype=torch.long) for f in feats]
            if cap:
                rows = [r[-cap:] if left else r[:cap] for r in rows]
            L = max(r.shape[0] for r in rows)
            out[f"{key}_input_ids"] = torch.stack([pad_to_length(r, L, self.pad, left) for r in rows])
            out[f"{key}_attention_mask"] = torch.stack(
                [pad_to_length(torch.ones_like(r), L, 0, left) for r in rows])
        for k in ("reference_chosen_logps", "reference_rejected_logps", "label", "margin"):
            if k in feats[0]:
                out[k] = torch.as_tensor([f[k] for f in feats])
        return out


@register_trainer_arguments("dpo")
@dataclass
class DPOConfig(TrainingArguments):
    trainer_prefix: str | None = "dpotrainer"
    beta: float = 0.1
    label_smoothing: float = 0.0
    loss_type: str = "sigmoid"
    use_weighting: bool = False
    reference_free: bool = False
    precompute_ref_log_probs: bool = False
    max_prompt_length: int | None = 512
    max_completion_length: int | None = None
    rpo_alpha: float | None = None
    discopop_tau: float = 0.05
    sync_ref_model: bool = False
    ref_model_mixup_alpha: float = 0.9
    ref_model_sync_steps: int = 64
    padding_value: int | None = None
    disable_dropout: bool = True


class _PreferenceBase(Trainer):
    """Shared: tokenise-free collation, frozen reference model, reward metrics."""

    needs_reference = True

    def __init__(self, arguments=None, model=None, reference_model=None, processing_class=None, train_dataset=None,
                 eval_dataset=None, data_collator=None, **kw):
        arguments = arguments or self.arguments_class()
        train_dataset = kw.pop("dataset_train", train_dataset)
        eval_dataset = kw.pop("dataset_eval", eval_dataset)
        tok = processing_class if processing_class is not None else kw.pop("tokenizer", None)
        pad = getattr(arguments, "padding_value", None)
        if pad is None:
            pad = getattr(tok, "pad_token_id", None) or 0
        self.pad_token_id = pad
        if data_collator is None:
            data_collator = self._default_collator(arguments)
        self.reference_model = reference_model
        super().__init__(arguments=arguments, model=model, dataset_train=train_dataset, dataset_eval=eval_dataset,
                         data_collator=data_collator, processing_class=tok, **kw)
        if self.needs_reference and self.reference_model is None and not getattr(arguments, "reference_free", False) \
                and not getattr(arguments, "precompute_ref_log_probs", False):
            self.reference_model = copy.deepcopy(self.model).eval().requires_grad_(False)

    def _default_collator(self, a):
        return DPODataCollator(self.pad_token_id, getattr(a, "max_prompt_length", None),
                               getattr(a, "max_completion_length", None))

    @torch.no_grad()
    def reference_logps(self, batch: dict) -> tuple[torch.Tensor, torch.Tensor]:
        if "reference_chosen_logps" in batch:
            return batch["reference_chosen_logps"].float(), batch["reference_rejected_logps"].float()
        if self.reference_model is None:
            z = torch.zeros(batch["chosen_input_ids"].shape[0], device=batch["chosen_input_ids"].device)
            return z, z
        r = concatenated_forward(self.reference_model, batch, pad_token_id=self.pad_token_id)
        return r["chosen_logps"].detach(), r["rejected_logps"].detach()

    @staticmethod
    def _reward_metrics(cr, rr, pc=None, pr=None) -> dict:
        m = {"rewards/chosen": cr.mean(), "rewards/rejected": rr.mean(), "rewards/accuracies": (cr > rr).float().mean(),
             "rewards/margins": (cr - rr).mean()}
        if pc is not None:
            m["logps/chosen"], m["logps/rejected"] = pc.detach().mean(), pr.detach().mean()
        return m

    def _maybe_sync_reference(self, step: int) -> None:
        a = self.arguments
        if getattr(a, "sync_ref_model", False) and self.reference_model is not None and \
                step % max(1, a.ref_model_sync_steps) == 0:
            al = a.ref_model_mixup_alpha
            with torch.no_grad():
                for pr, pp in zip(self.reference_model.parameters(), self.model.parameters()):
                    pr.mul_(al).add_(pp.detach().to(pr.dtype), alpha=1 - al)


@register_trainer("dpo")
class DPOTrainer(_PreferenceBase):
    trainer_type = "dpo"
    arguments_class = DPOConfig

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        pol = concatenated_forward(model, batch, pad_token_id=self.pad_token_id,
                                   want_nll=a.rpo_alpha is not None)
        rc, rr = self.reference_logps(batch)
        losses, cr, rrw = dpo_loss(pol["chosen_logps"], pol["rejected_logps"], rc, rr, beta=a.beta,
                                   label_smoothing=a.label_smoothing, loss_type=a.loss_type,
                                   reference_free=a.reference_free, discopop_tau=a.discopop_tau)
        loss = losses.mean()
        if a.rpo_alpha is not None:
            loss = loss + a.rpo_alpha * pol["nll"]
        if pol["aux_loss"] is not None and a.aux_loss_enabled:
            loss = loss + pol["aux_loss"]
        if is_train:
            self._maybe_sync_reference(self.model_state.step)
        return LossMetrics(loss=loss * loss_scale,
                           other_metrics=self._reward_metrics(cr, rrw, pol["chosen_logps"], pol["rejected_logps"]))

    @torch.no_grad()
    def precompute_reference_log_probs(self, dataset) -> list[dict]:
        """Adds ``reference_*_logps`` to every row (easydel .../dpo_trainer.py:356-436)."""
        rows = []
        bs = self.micro_batch_size
        for s in range(0, len(dataset), bs):
            feats = [dict(dataset[i]) for i in range(s, min(s + bs, len(dataset)))]
            batch = {k: v.to(self.device) for k, v in self.data_collator(feats).items()}
            r = concatenated_forward(self.reference_model or self.model, batch, pad_token_id=self.pad_token_id)
            for i, f in enumerate(feats):
                f["reference_chosen_logps"] = float(r["chosen_logps"][i])
                f["reference_rejected_logps"] = float(r["rejected_logps"][i])
                rows.append(f)
        return rows


# ----------------------------------------------------------------------------------------- ORPO
@register_trainer_arguments("orpo")
@dataclass
class ORPOConfig(TrainingArguments):
    trainer_prefix: str | None = "orpotrainer"
    beta: float = 0.1                    # weight (lambda) of the odds-ratio term
    max_prompt_length: int | None = 512
    max_completion_length: int | None = None
    padding_value: int | None = None
    disable_dropout: bool = True


def orpo_loss(chosen_avg: torch.Tensor, rejected_avg: torch.Tensor, nll: torch.Tensor, beta: float):
    """``nll - beta * log sigmoid(log odds ratio)`` on length-averaged log-probabilities."""
    log_odds = (chosen_avg - rejected_avg) - (torch.log1p(-torch.exp(chosen_avg).clamp_max(1 - 1e-6)) -
                                              torch.log1p(-torch.exp(rejected_avg).clamp_max(1 - 1e-6)))
    ratio = tF.logsigmoid(log_odds)
    return nll - beta * ratio.mean(), log_odds, ratio


@register_trainer("orpo")
class ORPOTrainer(_PreferenceBase):
    trainer_type = "orpo"
    arguments_class = ORPOConfig
    needs_reference = False

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        pol = concatenated_forward(model, batch, average=True, pad_token_id=self.pad_token_id, want_nll=True)
        loss, log_odds, ratio = orpo_loss(pol["chosen_avg"], pol["rejected_avg"], pol["nll"], a.beta)
        cr, rr = (a.beta * pol["chosen_avg"]).detach(), (a.beta * pol["rejected_avg"]).detach()
        om = self._reward_metrics(cr, rr, pol["chosen_logps"], pol["rejected_logps"])
        om.update({"log_odds_ratio": ratio.detach().mean(), "log_odds_chosen": log_odds.detach().mean(),
                   "nll_loss": pol["nll"].detach()})
        return LossMetrics(loss=loss * loss_scale, other_metrics=om)


# ----------------------------------------------------------------------------------------- CPO / SimPO
@register_trainer_arguments("cpo")
@dataclass
class CPOConfig(TrainingArguments):
    trainer_prefix: str | None = "cpotrainer"
    beta: float = 0.1
    label_smoothing: float = 0.0
    loss_type: str = "sigmoid"          # sigmoid | hinge | ipo | simpo | alphapo
    cpo_alpha: float = 1.0
    simpo_gamma: float = 0.5
    alpha: float = 0.0                  # AlphaPO reward-shape parameter
    max_prompt_length: int | None = 512
    max_completion_length: int | None = None
    padding_value: int | None = None
    disable_dropout: bool = True


def cpo_loss(pc, pr, *, beta, label_smoothing=0.0, loss_type="sigmoid", simpo_gamma=0.5, alpha=0.0):
    if loss_type == "alphapo" and alpha != 0.0:
        pc_r = (1 - torch.exp(-alpha * pc)) / alpha
        pr_r = (1 - torch.exp(-alpha * pr)) / alpha
        logits = pc_r - pr_r
    else:
        logits = pc - pr
    if loss_type in ("simpo", "alphapo"):
        logits = logits - simpo_gamma / beta
        losses = -tF.logsigmoid(beta * logits) * (1 - label_smoothing) - tF.logsigmoid(-beta * logits) * label_smoothing
    elif loss_type == "sigmoid":
        losses = -tF.logsigmoid(beta * logits) * (1 - label_smoothing) - tF.logsigmoid(-beta * logits) * label_smoothing
    elif loss_type == "hinge":
        losses = torch.relu(1 - beta * logits)
    elif loss_type == "ipo":
        losses = (logits - 1 / (2 * beta)) ** 2
    else:
        raise ValueError(f"unknown CPO loss_type {loss_type!r}")
    return losses, (beta * pc).detach(), (beta * pr).detach()


@register_trainer("cpo")
class CPOTrainer(_PreferenceBase):
    trainer_type = "cpo"
    arguments_class = CPOConfig
    needs_reference = False

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        avg = a.loss_type in ("ipo", "simpo", "alphapo")
        pol = concatenated_forward(model, batch, average=avg, pad_token_id=self.pad_token_id, want_nll=True)
        pc, pr = (pol["chosen_avg"], pol["rejected_avg"]) if avg else (pol["chosen_logps"], pol["rejected_logps"])
        losses, cr, rr = cpo_loss(pc, pr, beta=a.beta, label_smoothing=a.label_smoothing, loss_type=a.loss_type,
                                  simpo_gamma=a.simpo_gamma, alpha=a.alpha)
        loss = losses.mean()
        if a.loss_type != "simpo" and a.cpo_alpha:
            loss = loss + a.cpo_alpha * pol["nll"]
        om = self._reward_metrics(cr, rr, pol["chosen_logps"], pol["rejected_logps"])
        om["nll_loss"] = pol["nll"].detach()
        return LossMetrics(loss=loss * loss_scale, other_metrics=om)


# ----------------------------------------------------------------------------------------- KTO / BCO (unpaired)
class UnpairedCollator:
    """Rows: ``prompt_input_ids``, ``completion_input_ids``, ``label`` (True = desirable)."""

    def __init__(self, pad_token_id: int = 0, max_prompt_length=None, max_completion_length=None):
        self.pad, self.mp, self.mc = pad_token_id, max_prompt_length, max_completion_length

    def __call__(self, feats):
        out = {}
        for key, left, cap in (("prompt", True, self.mp), ("completion", False, self.mc)):
            rows = [torch.as_tensor(f[f"{key}_input_ids"], dtype=torch.long) for f in feats]
            if cap:
                rows = [r[-cap:] if left else r[:cap] for r in rows]
            L = max(r.shape[0] for r in rows)
            out[f"{key}_input_ids"] = torch.stack([pad_to_length(r, L, self.pad, left) for r in rows])
            out[f"{key}_attention_mask"] = torch.stack([pad_to_length(torch.ones_like(r), L, 0, left) for r in rows])
        out["label"] = torch.as_tensor([bool(f["label"]) for f in feats])
        return out


def _unpaired_logps(model, batch, shift_completions: int = 0):
    """Sequence log-prob of each completion given its prompt; ``shift_completions`` rolls completions across
    the batch (mismatched pairs estimate the KL term of KTO)."""
    c, cm = batch["completion_input_ids"], batch["completion_attention_mask"]
    if shift_completions:
        c, cm = torch.roll(c, shift_completions, 0), torch.roll(cm, shift_completions, 0)
    ids = torch.cat([batch["prompt_input_ids"], c], 1)
    att = torch.cat([batch["prompt_attention_mask"], cm], 1)
    lm = torch.cat([torch.zeros_like(batch["prompt_attention_mask"]), cm], 1)
    lp, _, _ = sequence_logprobs(model, ids, att, lm)
    return lp


@register_trainer_arguments("kto")
@dataclass
class KTOConfig(TrainingArguments):
    trainer_prefix: str | None = "ktotrainer"
    beta: float = 0.1
    desirable_weight: float = 1.0
    undesirable_weight: float = 1.0
    loss_type: str = "kto"               # kto | apo_zero_unpaired
    max_prompt_length: int | None = 512
    max_completion_length: int | None = None
    padding_value: int | None = None
    precompute_ref_log_probs: bool = False
    reference_free: bool = False
    disable_dropout: bool = True


def kto_loss(policy_lp, ref_lp, policy_kl_lp, ref_kl_lp, label, *, beta, desirable_weight=1.0,
             undesirable_weight=1.0, loss_type="kto"):
    kl = (policy_kl_lp - ref_kl_lp).mean().clamp_min(0).detach() if policy_kl_lp is not None else \
        torch.zeros((), device=policy_lp.device)
    lr = policy_lp - ref_lp
    lab = label.bool()
    if loss_type == "kto":
        des = 1 - torch.sigmoid(beta * (lr - kl))
        und = 1 - torch.sigmoid(beta * (kl - lr))
    else:  # apo_zero_unpaired
        des = 1 - torch.sigmoid(beta * lr)
        und = torch.sigmoid(beta * lr)
    losses = torch.where(lab, desirable_weight * des, undesirable_weight * und)
    return losses, (beta * lr).detach(), kl


@register_trainer("kto")
class KTOTrainer(_PreferenceBase):
    trainer_type = "kto"
    arguments_class = KTOConfig

    def _default_collator(self, a):
        return UnpairedCollator(self.pad_token_id, a.max_prompt_length, a.max_completion_length)

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        pol = _unpaired_logps(model, batch)
        use_kl = a.loss_type == "kto" and batch["label"].shape[0] > 1
        pol_kl = _unpaired_logps(model, batch, 1) if use_kl else None
        with torch.no_grad():
            refm = self.reference_model
            if refm is None:
                ref, ref_kl = torch.zeros_like(pol), (torch.zeros_like(pol) if use_kl else None)
            else:
                ref = _unpaired_logps(refm, batch)
                ref_kl = _unpaired_logps(refm, batch, 1) if use_kl else None
        losses, rewards, kl = kto_loss(pol, ref, pol_kl.detach() if pol_kl is not None else None, ref_kl,
                                       batch["label"], beta=a.beta, desirable_weight=a.desirable_weight,
                                       undesirable_weight=a.undesirable_weight, loss_type=a.loss_type)
        lab = batch["label"].bool()
        om = {"kl": kl, "rewards/chosen": (rewards * lab).sum() / lab.sum().clamp_min(1),
              "rewards/rejected": (rewards * ~lab).sum() / (~lab).sum().clamp_min(1)}
        return LossMetrics(loss=losses.mean() * loss_scale, other_metrics=om)


@register_trainer_arguments("bco")
@dataclass
class BCOConfig(TrainingArguments):
    trainer_prefix: str | None = "bcotrainer"
    beta: float = 0.1
    max_prompt_length: int | None = 512
    max_completion_length: int | None = None
    padding_value: int | None = None
    precompute_ref_log_probs: bool = False
    reference_free: bool = False
    delta_momentum: float = 0.9          # running mean of the reward used as the classifier threshold
    disable_dropout: bool = True


@register_trainer("bco")
class BCOTrainer(_PreferenceBase):
    """Binary-classifier optimisation: rewards ``beta * log(pi/ref)`` are pushed above / below a running mean."""

    trainer_type = "bco"
    arguments_class = BCOConfig

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.running_delta = 0.0
        self._delta_initialised = False

    def _default_collator(self, a):
        return UnpairedCollator(self.pad_token_id, a.max_prompt_length, a.max_completion_length)

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        pol = _unpaired_logps(model, batch)
        with torch.no_grad():
            ref = _unpaired_logps(self.reference_model, batch) if self.reference_model is not None else \
                torch.zeros_like(pol)
        rewards = a.beta * (pol - ref)
        lab = batch["label"].bool()
        if is_train:
            mean_r = float(rewards.detach().mean())
            if not self._delta_initialised:
                self.running_delta, self._delta_initialised = mean_r, True
            else:
                self.running_delta = a.delta_momentum * self.running_delta + (1 - a.delta_momentum) * mean_r
        d = self.running_delta
        losses = torch.where(lab, -tF.logsigmoid(rewards - d), -tF.logsigmoid(-(rewards - d)))
        rd = rewards.detach()
        om = {"delta": torch.tensor(d), "rewards/chosen": (rd * lab).sum() / lab.sum().clamp_min(1),
              "rewards/rejected": (rd * ~lab).sum() / (~lab).sum().clamp_min(1)}
        return LossMetrics(loss=losses.mean() * loss_scale, other_metrics=om)


# ----------------------------------------------------------------------------------------- reward model
@register_trainer_arguments("reward")
@dataclass
class RewardConfig(TrainingArguments):
    trainer_prefix: str | None = "rewardtrainer"
    center_rewards_coefficient: float | None = None
    padding_value: int | None = None
    disable_dropout: bool = True


class RewardCollator:
    """Rows: ``input_ids_chosen``, ``input_ids_rejected`` (+ optional ``margin``)."""

    def __init__(self, pad_token_id: int = 0, max_length: int | None = None):
        self.pad, self.max_length = pad_token_id, max_length

    def __call__(self, feats):
        out = {}
        for key in ("chosen", "rejected"):
            rows = [torch.as_tensor(f[f"input_ids_{key}"], dtype=torch.long)[: self.max_length] for f in feats]
            L = max(r.shape[0] for r in rows)
            out[f"input_ids_{key}"] = torch.stack([pad_to_length(r, L, self.pad) for r in rows])
            out[f"attention_mask_{key}"] = torch.stack([pad_to_length(torch.ones_like(r), L, 0) for r in rows])
        if "margin" in feats[0]:
            out["margin"] = torch.as_tensor([float(f["margin"]) for f in feats])
        return out


@register_trainer("reward")
class RewardTrainer(Trainer):
    """Bradley-Terry pairwise loss on a sequence-classification model with one label
    (easydel/trainers/reward_trainer)."""

    trainer_type = "reward"
    arguments_class = RewardConfig

    def __init__(self, arguments=None, model=None, processing_class=None, train_dataset=None, eval_dataset=None,
                 data_collator=None, **kw):
        arguments = arguments or RewardConfig()
        tok = processing_class if processing_class is not None else kw.pop("tokenizer", None)
        pad = arguments.padding_value if arguments.padding_value is not None else (getattr(tok, "pad_token_id", 0) or 0)
        super().__init__(arguments=arguments, model=model, dataset_train=kw.pop("dataset_train", train_dataset),
                         dataset_eval=kw.pop("dataset_eval", eval_dataset),
                         data_collator=data_collator or RewardCollator(pad, arguments.max_length),
                         processing_class=tok, **kw)

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        ids = torch.cat([_pad_cols(batch["input_ids_chosen"], batch["input_ids_rejected"]),
                         _pad_cols(batch["input_ids_rejected"], batch["input_ids_chosen"])], 0)
        att = torch.cat([_pad_cols(batch["attention_mask_chosen"], batch["attention_mask_rejected"]),
                         _pad_cols(batch["attention_mask_rejected"], batch["attention_mask_chosen"])], 0)
        r = model(input_ids=ids, attention_mask=att).logits.float()[:, 0]
        B = batch["input_ids_chosen"].shape[0]
        rc, rr = r[:B], r[B:]
        diff = rc - rr - (batch["margin"].to(rc) if "margin" in batch else 0.0)
        loss = -tF.logsigmoid(diff).mean()
        coef = self.arguments.center_rewards_coefficient
        if coef:
            loss = loss + coef * ((rc + rr) ** 2).mean()
        return LossMetrics(loss=loss * loss_scale, accuracy=(rc > rr).float().mean().detach(),
                           other_metrics={"rewards/chosen": rc.detach().mean(), "rewards/rejected": rr.detach().mean()})


def _pad_cols(t: torch.Tensor, other: torch.Tensor) -> torch.Tensor:
    L = max(t.shape[1], other.shape[1])
    if t.shape[1] == L:
        return t
    return torch.cat([t, torch.zeros(t.shape[0], L - t.shape[1], dtype=t.dtype, device=t.device)], 1)
