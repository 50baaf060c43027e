"""PPO (value head + GAE) and the online preference trainers XPO and Nash-MD.

Reference: easydel/trainers/proximal_policy_optimization_trainer (value head, GAE, clipped policy / value losses),
xpo_trainer (online DPO with an optimism bonus on reference samples), nash_md_trainer (samples from the geometric
mixture of policy and reference, REINFORCE on the preference probability with a KL regulariser).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

import torch
import torch.nn.functional as tF
from torch import nn

from ..infra.loss_utils import LossMetrics
from ._logprob_utils import token_logprobs
from .rl import GRPOConfig, GRPOTrainer
from .training_configurations import register_trainer, register_trainer_arguments


# ----------------------------------------------------------------------------------------- PPO
@register_trainer_arguments("ppo")
@dataclass
class PPOConfig(GRPOConfig):
    trainer_prefix: str | None = "ppotrainer"
    num_return_sequences: int = 1
    kl_coef: float = 0.05
    cliprange: float = 0.2
    cliprange_value: float = 0.2
    vf_coef: float = 0.1
    gamma: float = 1.0
    lam: float = 0.95
    whiten_rewards: bool = False
    whiten_advantages: bool = True
    missing_eos_penalty: float | None = None
    beta: float = 0.0


class ValueHead(nn.Module):
    """Scalar value per position from the backbone's last hidden state
    (easydel/trainers/proximal_policy_optimization_trainer value head)."""

    def __init__(self, hidden_size: int, dtype=torch.float32):
        super().__init__()
        self.summary = nn.Linear(hidden_size, 1, dtype=dtype)
        nn.init.normal_(self.summary.weight, std=1.0 / (hidden_size + 1) ** 0.5)
        nn.init.zeros_(self.summary.bias)

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.summary(hidden.to(self.summary.weight.dtype))[..., 0].float()


def gae(rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, gamma: float, lam: float):
    """Generalised advantage estimation over ``[N, T]`` token rewards; positions outside ``mask`` carry nothing."""
    N, T = rewards.shape
    adv = torch.zeros_like(rewards)
    last = torch.zeros(N, device=rewards.device)
    for t in reversed(range(T)):
        nxt = values[:, t + 1] * mask[:, t + 1] if t + 1 < T else torch.zeros(N, device=rewards.device)
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = (delta + gamma * lam * last) * mask[:, t]
        adv[:, t] = last
    return adv, adv + values


def _whiten(x, mask, shift_mean=True):
    mean = (x * mask).sum() / mask.sum().clamp_min(1)
    var = ((x - mean) ** 2 * mask).sum() / mask.sum().clamp_min(1)
    y = (x - mean) * torch.rsqrt(var + 1e-8)
    return y if shift_mean else y + mean


@register_trainer("ppo")
class PPOTrainer(GRPOTrainer):
    trainer_type = "ppo"
    arguments_class = PPOConfig

    def __init__(self, arguments=None, model=None, reward_funcs=None, reward_model=None, value_model=None, **kw):
        arguments = arguments or PPOConfig()
        hidden = model.config.hidden_size
        if not hasattr(model, "value_head"):
            model.value_head = ValueHead(hidden, torch.float32).to(model.device)
        fns = reward_funcs if reward_funcs is not None else reward_model
        super().__init__(arguments=arguments, model=model, reward_funcs=fns, **kw)
        if self.reference_model is None and arguments.kl_coef:
            self.reference_model = copy.deepcopy(self.model).eval().requires_grad_(False)

    def _advantages(self, rewards, comp_mask, n):
        return rewards, {}     # token-level credit comes from GAE in `_extra_rollout_tensors`

    @torch.no_grad()
    def _values(self, ids, att):
        out = self.model(input_ids=ids, attention_mask=att, apply_lm_head=False)
        return self.model.value_head(out.last_hidden_state)[:, :-1]

    def _extra_rollout_tensors(self, batch, new, comp, cmask, rewards, n):
        a = self.arguments
        ids, att, lm = new["input_ids"], new["attention_mask"], new["loss_mask"]
        m = lm[:, 1:].float()
        old = new["old_logps"]
        with torch.no_grad():
            was = self.model.training
            self.model.eval()
            values = self._values(ids, att) * m
            ref = self._chunked_logps(self.reference_model, ids, att, lm) if self.reference_model is not None else old
            self.model.train(was)
        scores = rewards.clone()
        if a.missing_eos_penalty is not None:
            eos = self._eos_ids()
            if eos:
                has = torch.isin(comp, torch.tensor(eos, device=comp.device)).any(1)
                scores = scores - a.missing_eos_penalty * (~has).float()
        tok_r = -a.kl_coef * (old - ref) * m
        last = (m.cumsum(1) == m.sum(1, keepdim=True)) & (m > 0)
        tok_r = tok_r + last.float() * scores[:, None]
        if a.whiten_rewards:
            tok_r = _whiten(tok_r, m, shift_mean=False) * m
        adv, ret = gae(tok_r, values, torch.cat([m, torch.zeros_like(m[:, :1])], 1), a.gamma, a.lam)
        if a.whiten_advantages:
            adv = _whiten(adv, m) * m
        return {"token_advantages": adv, "returns": ret * m, "old_values": values,
                "advantages": torch.zeros(ids.shape[0], device=self.device)}

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        lp, m, _, out = token_logprobs(model, batch["input_ids"], batch["attention_mask"], batch["loss_mask"],
                                       temperature=a.temperature)
        v = model.value_head(out.last_hidden_state)[:, :-1]
        adv, ret, v_old = batch["token_advantages"], batch["returns"], batch["old_values"]
        ratio = torch.exp(lp - batch["old_logps"])
        pg = torch.maximum(-adv * ratio, -adv * ratio.clamp(1 - a.cliprange, 1 + a.cliprange))
        v_clip = torch.maximum(torch.minimum(v, v_old + a.cliprange_value), v_old - a.cliprange_value)
        vf = 0.5 * torch.maximum((v - ret) ** 2, (v_clip - ret) ** 2)
        den = m.sum().clamp_min(1)
        pg_loss, vf_loss = (pg * m).sum() / den, (vf * m).sum() / den
        stats = {"ppo/policy_loss": pg_loss.detach(), "ppo/value_loss": vf_loss.detach(),
                 "ppo/approx_kl": (0.5 * ((lp - batch["old_logps"]) ** 2).detach() * m).sum() / den,
                 "ppo/clip_fraction": (((ratio - 1).abs() > a.cliprange).float() * m).sum() / den}
        return LossMetrics(loss=(pg_loss + a.vf_coef * vf_loss) * loss_scale, other_metrics=stats)


# ----------------------------------------------------------------------------------------- online preference base
class _OnlinePairTrainer(GRPOTrainer):
    """Two completions per prompt (policy vs. opponent), ranked by the reward functions or a pairwise judge."""

    def __init__(self, arguments=None, model=None, reward_funcs=None, judge=None, **kw):
        self.judge = judge
        if reward_funcs is None and judge is None:
            raise ValueError("pass `reward_funcs` (or a reward model) or a pairwise `judge`")
        super().__init__(arguments=arguments, model=model, reward_funcs=reward_funcs or (lambda **k: [0.0]), **kw)
        if self.reference_model is None:
            self.reference_model = copy.deepcopy(self.model).eval().requires_grad_(False)

    def _opponent_completions(self, p_ids, p_mask):
        return self.sample_completions(p_ids, p_mask, 1, model=self.reference_model)

    def _preference(self, p_ids, p_mask, c1, m1, c2, m2, extras):
        """P(first beats second) per prompt."""
        if self.judge is not None:
            prompts = self._decode(p_ids, p_mask)
            probs = self.judge(prompts, list(zip(self._decode(c1, m1), self._decode(c2, m2))))
            return torch.as_tensor(probs, dtype=torch.float32, device=self.device)
        r1, _ = self.score(p_ids, p_mask, c1, m1, extras, 1)
        r2, _ = self.score(p_ids, p_mask, c2, m2, extras, 1)
        return torch.sigmoid(r1 - r2)

    def _pack(self, p_ids, p_mask, comp, cmask):
        ids = torch.cat([p_ids.to(self.device), comp], 1)
        att = torch.cat([p_mask.to(self.device), cmask], 1)
        lm = torch.cat([torch.zeros_like(p_mask).to(self.device), cmask], 1)
        return ids, att, lm


# ----------------------------------------------------------------------------------------- XPO
@register_trainer_arguments("xpo")
@dataclass
class XPOConfig(GRPOConfig):
    trainer_prefix: str | None = "xpotrainer"
    num_return_sequences: int = 1
    beta: float = 0.1
    alpha: float = 1e-5
    loss_type: str = "sigmoid"      # sigmoid | ipo


@register_trainer("xpo")
class XPOTrainer(_OnlinePairTrainer):
    """Exploratory preference optimisation: DPO on (policy sample, reference sample) pairs ranked online, plus
    ``alpha * log pi(y_ref | x)`` which pushes probability away from what the reference already produces."""

    trainer_type = "xpo"
    arguments_class = XPOConfig

    def _preprocess_batch_input(self, state, batch, is_train):
        p_ids, p_mask = batch["input_ids"], batch["attention_mask"]
        extras = {k: v for k, v in batch.items() if k not in ("input_ids", "attention_mask")}
        c_pol, m_pol = self.sample_completions(p_ids, p_mask, 1)
        c_ref, m_ref = self._opponent_completions(p_ids, p_mask)
        pref = self._preference(p_ids, p_mask, c_pol, m_pol, c_ref, m_ref, extras)
        pol_wins = pref >= 0.5
        new = {"policy_wins": pol_wins}
        for name, (c, m) in (("pol", (c_pol, m_pol)), ("ref", (c_ref, m_ref))):
            ids, att, lm = self._pack(p_ids, p_mask, c, m)
            new[f"{name}_ids"], new[f"{name}_att"], new[f"{name}_lm"] = ids, att, lm
            with torch.no_grad():
                new[f"{name}_reflp"] = self._chunked_logps(self.reference_model, ids, att, lm).sum(1)
        return new, {"xpo/policy_win_rate": float(pol_wins.float().mean())}

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        lp_pol = token_logprobs(model, batch["pol_ids"], batch["pol_att"], batch["pol_lm"])[0].sum(1)
        lp_ref = token_logprobs(model, batch["ref_ids"], batch["ref_att"], batch["ref_lm"])[0].sum(1)
        w = batch["policy_wins"]
        chosen = torch.where(w, lp_pol, lp_ref)
        rejected = torch.where(w, lp_ref, lp_pol)
        chosen_ref = torch.where(w, batch["pol_reflp"], batch["ref_reflp"])
        rejected_ref = torch.where(w, batch["ref_reflp"], batch["pol_reflp"])
        logits = (chosen - chosen_ref) - (rejected - rejected_ref)
        if a.loss_type == "ipo":
            dpo = (logits - 1 / (2 * a.beta)) ** 2
        else:
            dpo = -tF.logsigmoid(a.beta * logits)
        xpo = a.alpha * lp_ref
        loss = (dpo + xpo).mean()
        stats = {"xpo/dpo_loss": dpo.detach().mean(), "xpo/optimism": xpo.detach().mean(),
                 "rewards/margins": (a.beta * logits).detach().mean()}
        return LossMetrics(loss=loss * loss_scale, other_metrics=stats)


# ----------------------------------------------------------------------------------------- Nash-MD
@register_trainer_arguments("nash-md")
@dataclass
class NashMDConfig(GRPOConfig):
    trainer_prefix: str | None = "nashmdtrainer"
    num_return_sequences: int = 1
    beta: float = 0.1
    mixture_coef: float = 0.5


@register_trainer("nash-md")
class NashMDTrainer(_OnlinePairTrainer):
    trainer_type = "nash-md"
    arguments_class = NashMDConfig

    @torch.no_grad()
    def _opponent_completions(self, p_ids, p_mask):
        """Samples from ``softmax((1 - c) * logits_policy + c * logits_ref)`` token by token."""
        a = self.arguments
        dev = self.device
        ids, att = p_ids.to(dev), p_mask.to(dev)
        B, T = ids.shape
        C = a.max_completion_length
        models = (self.model, self.reference_model)
        was = self.model.training
        self.model.eval()
        caches = [m.init_cache(B, T + C) for m in models]
        pos = (att.long().cumsum(-1) - 1).clamp_min(0)
        meta = None
        if not bool(att.all()):
            seg = torch.ones(B, T + C, dtype=torch.int32, device=dev)
            seg[:, :T] = att.to(torch.int32)
            meta = {"kv_segment_ids": seg}
        logits = []
        for m, c in zip(models, caches):
            o = m(input_ids=ids, position_ids=pos, past_key_values=c, cache_metadata=meta)
            c.advance(T)
            logits.append(o.logits[:, -1].float())
        nxt = pos[:, -1] + 1
        toks = []
        g = torch.Generator(device=dev).manual_seed(int(self.model_state.step) * 104729 + 17)
        for step in range(C):
            mix = ((1 - a.mixture_coef) * logits[0] + a.mixture_coef * logits[1]) / max(a.temperature, 1e-5)
            tok = torch.multinomial(torch.softmax(mix, -1), 1, generator=g)[:, 0]
            toks.append(tok)
            if step == C - 1:
                break
            logits = []
            for m, c in zip(models, caches):
                o = m(input_ids=tok[:, None], position_ids=nxt[:, None], past_key_values=c, cache_metadata=meta)
                c.advance(1)
                logits.append(o.logits[:, -1].float())
            nxt = nxt + 1
        self.model.train(was)
        comp = torch.stack(toks, 1)
        from .rl import first_eos_mask

        return comp, first_eos_mask(comp, self._eos_ids())

    def _preprocess_batch_input(self, state, batch, is_train):
        p_ids, p_mask = batch["input_ids"], batch["attention_mask"]
        extras = {k: v for k, v in batch.items() if k not in ("input_ids", "attention_mask")}
        c_pol, m_pol = self.sample_completions(p_ids, p_mask, 1)
        c_mix, m_mix = self._opponent_completions(p_ids, p_mask)
        prob = self._preference(p_ids, p_mask, c_pol, m_pol, c_mix, m_mix, extras)
        ids, att, lm = self._pack(p_ids, p_mask, c_pol, m_pol)
        with torch.no_grad():
            ref_lp = self._chunked_logps(self.reference_model, ids, att, lm)
        return ({"input_ids": ids, "attention_mask": att, "loss_mask": lm, "ref_logps": ref_lp,
                 "preference": prob}, {"nash_md/win_probability": float(prob.mean())})

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        lp, m, _, _ = token_logprobs(model, batch["input_ids"], batch["attention_mask"], batch["loss_mask"])
        seq = lp.sum(1)
        score = (batch["preference"] - 0.5) * seq
        log_ratio = (lp - batch["ref_logps"]).detach()
        kl_loss = (log_ratio * lp).sum(1)
        loss = (a.beta * kl_loss - score).mean()
        stats = {"nash_md/kl": (log_ratio * m).sum(1).mean(), "nash_md/score": score.detach().mean()}
        return LossMetrics(loss=loss * loss_scale, other_metrics=stats)
