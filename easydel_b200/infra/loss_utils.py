"""Loss configuration, metrics container and task losses.

API follows easydel/infra/loss_utils.py (``LossConfig`` :346, ``LossMetrics`` :439, task losses
:2605-2885, ``auxiliary_load_balancing_loss_func`` :1760). The causal-LM loss never materialises
``[tokens, vocab]`` logits when it is handed hidden states plus the LM-head weight: it runs the
chunked LM-head + cross-entropy op (``ops.functional.linear_cross_entropy``).
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass, field, fields

import torch
import torch.nn.functional as tF

from ..ops import functional as F
from ..ops import reference as R


class SpecialLossNormalizingFactor:
    NUM_REAL_TARGET_TOKENS = "NUM_REAL_TARGET_TOKENS"
    NUM_TOTAL_TARGET_TOKENS = "NUM_TOTAL_TARGET_TOKENS"
    AVERAGE_PER_SEQUENCE = "AVERAGE_PER_SEQUENCE"
    NO_WEIGHT_NUM_REAL_TARGET_TOKENS = "NO_WEIGHT_NUM_REAL_TARGET_TOKENS"


@dataclass
class LossConfig:
    ignore_index: int = -100
    label_smoothing: float = 0.0
    z_loss: float = 0.0
    loss_normalizing_factor: tp.Any = "NUM_REAL_TARGET_TOKENS"
    num_labels: int | None = None
    problem_type: str | None = None
    divide_weight_sum: bool = False
    shift_tokens: bool = True
    break_on_nan: bool = True
    reduction: str | None = None
    num_classification_labels: int | None = None
    classification_problem_type: str | None = None
    chunk_vocab_size: int | None = None
    chunk_token_size: int | None = None
    chunk_block_size: int | None = 4096
    compute_dtype: str | None = None

    def __repr__(self):
        return type(self).__name__ + "(\n" + "\n".join(f"    {f.name}: {getattr(self, f.name)!r}"
                                                      for f in fields(self)) + "\n)"

    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}


@dataclass
class LossMetrics:
    loss: torch.Tensor | float | None = None
    z_loss: torch.Tensor | float | None = None
    weight_sum: torch.Tensor | float | None = None
    accuracy: torch.Tensor | float | None = None
    learning_rate: torch.Tensor | float | None = None
    max_grad_norm: torch.Tensor | float | None = None
    mean_grad_norm: torch.Tensor | float | None = None
    grad_norms: tp.Any = None
    chosen_rewards: torch.Tensor | None = None
    rejected_rewards: torch.Tensor | None = None
    other_metrics: dict | None = None
    execution_time: float | None = None

    def to_float_dict(self) -> dict[str, float]:
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            if v is None or f.name in ("grad_norms", "other_metrics"):
                continue
            try:
                out[f.name] = float(v.detach().float().mean().item()) if isinstance(v, torch.Tensor) else float(v)
            except (TypeError, ValueError):
                continue
        for k, v in (self.other_metrics or {}).items():
            try:
                out[k] = float(v.detach().float().mean().item()) if isinstance(v, torch.Tensor) else float(v)
            except (TypeError, ValueError):
                continue
        return out


def _normalizer(cfg: LossConfig, labels: torch.Tensor, n_valid: torch.Tensor):
    f = cfg.loss_normalizing_factor
    if isinstance(f, (int, float)) and not isinstance(f, bool):
        return float(f)
    name = str(getattr(f, "name", f)).upper()
    if name in ("NUM_REAL_TARGET_TOKENS", "NO_WEIGHT_NUM_REAL_TARGET_TOKENS"):
        return None  # = n_valid (handled by the op)
    if name == "NUM_TOTAL_TARGET_TOKENS":
        return float(labels.numel())
    if name == "AVERAGE_PER_SEQUENCE":
        return None
    raise ValueError(f"unknown loss_normalizing_factor {f!r}")


def causal_lm_loss_from_hidden(hidden: torch.Tensor, lm_head_weight: torch.Tensor, labels: torch.Tensor,
                               config: LossConfig | None = None, *, lm_head_bias=None, softcap: float = 0.0,
                               chunk_size: int | None = None, loss_scale: float = 1.0,
                               want_accuracy: bool = True, already_shifted: bool = False,
                               count_group=None) -> LossMetrics:
    """Shifted next-token CE from final hidden states ``[B,T,H]`` and labels ``[B,T]``.

    ``loss_scale`` multiplies the result (the trainer passes ``1 / gradient_accumulation_steps``).
    ``count_group``: ``hidden`` / ``labels`` are this rank's rows of a token axis sharded over that process
    group; the token count that normalises the loss (and the accuracy) is then the group's, so the ranks' losses
    add up to the loss of the whole batch. ``already_shifted``: row t of ``labels`` is the target of row t.
    """
    cfg = config or LossConfig()
    if cfg.shift_tokens and not already_shifted:
        # keep T rows (row t predicts label t+1; the last row is ignored) so no activation copy is needed
        shifted = torch.full_like(labels, cfg.ignore_index)
        shifted[..., :-1] = labels[..., 1:]
        labels = shifted
    norm = _normalizer(cfg, labels, None)
    red_scale = None
    if norm is not None:
        if count_group is not None and str(getattr(cfg.loss_normalizing_factor, "name",
                                                   cfg.loss_normalizing_factor)).upper() == "NUM_TOTAL_TARGET_TOKENS":
            import torch.distributed as dist

            norm = norm * dist.get_world_size(count_group)   # the labels seen here are one rank's rows
        red_scale = loss_scale / norm
    loss, n_valid, acc = F.linear_cross_entropy(
        hidden.reshape(-1, hidden.shape[-1]), lm_head_weight, labels.reshape(-1), bias=lm_head_bias,
        ignore_index=cfg.ignore_index, label_smoothing=cfg.label_smoothing, z_loss=cfg.z_loss, softcap=softcap,
        chunk_size=chunk_size or cfg.chunk_token_size or 2048, reduction_scale=red_scale,
        loss_scale=loss_scale, want_accuracy=want_accuracy, count_group=count_group)
    if count_group is not None and want_accuracy:
        import torch.distributed as dist

        acc = acc.detach().clone()
        dist.all_reduce(acc, group=count_group)   # each rank counted its correct rows over the group's total
    return LossMetrics(loss=loss, weight_sum=n_valid, accuracy=acc if want_accuracy else None)


def ForCausalLMLoss(logits: torch.Tensor, labels: torch.Tensor, attention_mask: torch.Tensor | None = None,
                    config: LossConfig | None = None, **_) -> LossMetrics:
    """CE over materialised logits ``[B,T,V]`` (kept for heads / trainers that need the logits anyway)."""
    cfg = config or LossConfig()
    if cfg.shift_tokens:
        logits = logits[..., :-1, :]
        labels = labels[..., 1:]
        if attention_mask is not None:
            attention_mask = attention_mask[..., 1:]
    if attention_mask is not None:
        labels = torch.where(attention_mask.bool(), labels, torch.full_like(labels, cfg.ignore_index))
    per, lse = R.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1),
                               ignore_index=cfg.ignore_index, label_smoothing=cfg.label_smoothing, z_loss=cfg.z_loss)
    valid = (labels.reshape(-1) != cfg.ignore_index)
    n = valid.sum().clamp_min(1).to(torch.float32)
    norm = _normalizer(cfg, labels, n)
    loss = per.sum() / (n if norm is None else norm)
    acc = ((logits.reshape(-1, logits.shape[-1]).argmax(-1) == labels.reshape(-1)) & valid).sum() / n
    zl = (cfg.z_loss * lse.pow(2) * valid).sum() / n if cfg.z_loss else None
    return LossMetrics(loss=loss, z_loss=zl, weight_sum=n, accuracy=acc)


def ForSequenceClassificationLoss(logits: torch.Tensor, labels: torch.Tensor, config: LossConfig | None = None,
                                  **_) -> LossMetrics:
    cfg = config or LossConfig()
    num_labels = cfg.num_labels or cfg.num_classification_labels or logits.shape[-1]
    problem = cfg.problem_type or cfg.classification_problem_type
    if problem is None:
        if num_labels == 1:
            problem = "regression"
        elif labels.dtype in (torch.long, torch.int32, torch.int64):
            problem = "single_label_classification"
        else:
            problem = "multi_label_classification"
    if problem == "regression":
        loss = tF.mse_loss(logits.float().squeeze(-1), labels.float().squeeze(-1))
        acc = None
    elif problem == "single_label_classification":
        loss = tF.cross_entropy(logits.float().view(-1, num_labels), labels.view(-1),
                                label_smoothing=cfg.label_smoothing)
        acc = (logits.argmax(-1).view(-1) == labels.view(-1)).float().mean()
    else:
        loss = tF.binary_cross_entropy_with_logits(logits.float(), labels.float())
        acc = ((logits > 0) == (labels > 0.5)).float().mean()
    return LossMetrics(loss=loss, accuracy=acc)


def ForQuestionAnsweringLoss(start_logits, end_logits, start_positions, end_positions, config=None, **_):
    ign = start_logits.shape[-1]
    sp = start_positions.clamp(0, ign)
    ep = end_positions.clamp(0, ign)
    ls = tF.cross_entropy(start_logits.float(), sp, ignore_index=ign)
    le = tF.cross_entropy(end_logits.float(), ep, ignore_index=ign)
    return LossMetrics(loss=(ls + le) / 2)


def ForTokenClassification(logits, labels, config: LossConfig | None = None, **_):
    cfg = config or LossConfig()
    loss = tF.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.view(-1),
                            ignore_index=cfg.ignore_index)
    return LossMetrics(loss=loss)


def auxiliary_load_balancing_loss_func(gate_logits, num_experts: int, top_k: int,
                                       attention_mask: torch.Tensor | None = None) -> torch.Tensor:
    """Load-balancing loss over a tuple of per-layer router logits ``[T, E]`` (HF / reference semantics)."""
    from ..layers.moe import load_balancing_loss

    if gate_logits is None:
        return torch.zeros(())
    if isinstance(gate_logits, (tuple, list)):
        logits = torch.cat([g.reshape(-1, g.shape[-1]) for g in gate_logits], dim=0)
        n_layers = len(gate_logits)
    else:
        logits, n_layers = gate_logits.reshape(-1, gate_logits.shape[-1]), 1
    probs = torch.softmax(logits.float(), dim=-1)
    idx = probs.topk(top_k, dim=-1).indices
    mask = None
    if attention_mask is not None:
        mask = attention_mask.reshape(-1).repeat(n_layers)
    return load_balancing_loss(probs, idx, num_experts, mask)


LOSS_MAPPING = {
    "ForCausalLM": ForCausalLMLoss,
    "ForSequenceClassification": ForSequenceClassificationLoss,
    "ForQuestionAnswering": ForQuestionAnsweringLoss,
    "ForTokenClassification": ForTokenClassification,
}


# the functional variants and the strategy objects live in their own module and are part of this one's surface
from .loss_functions import (SLNF, BaseLossStrategy, CausalLMLossStrategy, FunctionalLossStrategy,  # noqa: E402,F401
                             LossForwardPlan, compute_weighted_cross_entropy,
                             compute_weighted_cross_entropy_and_accuracy,
                             convert_special_loss_normalizing_factor_to_enum, cross_entropy_blockwise_logits,
                             cross_entropy_loss_and_accuracy, cross_entropy_with_logits, dynamic_cross_entropy_loss,
                             fixed_cross_entropy, get_factor_and_weight, onehot, resolve_loss_strategy,
                             sigmoid_cross_entropy_with_logits, sparse_cross_entropy_chunked_tokens,
                             sparse_cross_entropy_chunked_vocab)
