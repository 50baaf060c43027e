"""Functional cross-entropy variants and loss strategies.

The public helpers of easydel/infra/loss_utils.py beyond the task losses: sigmoid / softmax cross entropy with the
auxiliary z-loss, weighted and label-smoothed cross entropy with accuracy, vocabulary- and token-chunked sparse cross
entropy (memory-bounded forms), the normalising-factor resolver of packed batches, and the two-stage loss strategies
(``plan_forward`` tells the model what the loss needs, e.g. "skip the LM head", ``compute`` consumes the outputs).
All of it is plain tensor code in fp32; on CUDA the trainers' hot path stays the fused LM-head + cross-entropy kernel
(``ops.functional.linear_cross_entropy``), which these functions are tested against.
"""

from __future__ import annotations

import dataclasses
import typing as tp

import torch


class SLNF:
    """Special loss normalising factors (easydel/infra/loss_utils.py:302)."""

    NO_WEIGHT_NUM_REAL_TARGET_TOKENS_DIVIDE_BY_NUM_SEQUENCES = "NO_WEIGHT_NUM_REAL_TARGET_TOKENS_DIVIDE_BY_NUM_SEQUENCES"
    NUM_REAL_TARGET_TOKENS = "NUM_REAL_TARGET_TOKENS"
    NUM_TOTAL_TARGET_TOKENS = "NUM_TOTAL_TARGET_TOKENS"
    AVERAGE_PER_SEQUENCE = "AVERAGE_PER_SEQUENCE"
    ALL = (NO_WEIGHT_NUM_REAL_TARGET_TOKENS_DIVIDE_BY_NUM_SEQUENCES, NUM_REAL_TARGET_TOKENS, NUM_TOTAL_TARGET_TOKENS,
           AVERAGE_PER_SEQUENCE)


def convert_special_loss_normalizing_factor_to_enum(x: str) -> str:
    name = str(getattr(x, "value", x)).upper()
    if name not in SLNF.ALL:
        raise ValueError(f"unknown loss normalising factor {x!r}; known: {SLNF.ALL}")
    return name


def onehot(labels: torch.Tensor, num_classes: int, on_value: float = 1.0, off_value: float = 0.0) -> torch.Tensor:
    out = torch.full((*labels.shape, num_classes), off_value, dtype=torch.float32, device=labels.device)
    return out.scatter_(-1, labels.long().clamp(0, num_classes - 1)[..., None], on_value)


def sigmoid_cross_entropy_with_logits(logits: torch.Tensor, labels: torch.Tensor, weights=None,
                                      label_smoothing: float = 0.0) -> torch.Tensor:
    """Element-wise binary cross entropy on logits, numerically stable: ``max(x, 0) - x z + log1p(exp(-|x|))``."""
    x, z = logits.float(), labels.float()
    if label_smoothing:
        z = z * (1.0 - label_smoothing) + 0.5 * label_smoothing
    loss = x.clamp_min(0) - x * z + torch.log1p(torch.exp(-x.abs()))
    return loss if weights is None else loss * weights.float()


def cross_entropy_with_logits(logits: torch.Tensor, targets: torch.Tensor, z_loss: float = 0.0):
    """Soft-target cross entropy with the auxiliary z-loss ``z_loss * logsumexp(logits)^2``.

    ``targets`` are probabilities ``[..., V]``. Returns ``(loss + z term, z term)`` per position."""
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    ce = (targets.float() * (lse[..., None] - lf)).sum(-1)
    z = z_loss * lse.pow(2)
    return ce + z, z


def compute_weighted_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, weights: torch.Tensor | None = None,
                                   label_smoothing: float = 0.0, z_loss: float = 0.0,
                                   loss_normalizing_factor: float | None = None):
    """Label-smoothed cross entropy with z-loss over integer ``targets``.

    The smoothed target puts ``1 - label_smoothing`` on the label and spreads the rest over the other classes; the
    entropy of that target is subtracted so that a perfect prediction scores zero. Returns
    ``(sum of weighted losses [/ factor], sum of z terms [/ factor], weight sum)``."""
    V = logits.shape[-1]
    conf = 1.0 - label_smoothing
    low = label_smoothing / max(1, V - 1)
    soft = onehot(targets, V, conf, low)
    norm_const = -(conf * torch.log(torch.tensor(conf)) + (V - 1) * low * torch.log(torch.tensor(low + 1e-20)))
    total, z = cross_entropy_with_logits(logits, soft, z_loss)
    total = total - norm_const.to(total.device)
    if weights is not None:
        w = weights.float()
        total, z = total * w, z * w
        weight_sum = w.sum()
    else:
        weight_sum = torch.tensor(float(targets.numel()), device=logits.device)
    total, z = total.sum(), z.sum()
    if loss_normalizing_factor is not None:
        total, z = total / loss_normalizing_factor, z / loss_normalizing_factor
    return total, z, weight_sum


def compute_weighted_cross_entropy_and_accuracy(logits, targets, weights=None, label_smoothing: float = 0.0,
                                                z_loss: float = 0.0, loss_normalizing_factor: float | None = None):
    """As :func:`compute_weighted_cross_entropy` plus the weighted accuracy. Returns
    ``(loss, z_loss, weight_sum, accuracy)``."""
    total, z, weight_sum = compute_weighted_cross_entropy(logits, targets, weights, label_smoothing, z_loss,
                                                          loss_normalizing_factor)
    hit = (logits.argmax(-1) == targets).float()
    if weights is not None:
        hit = hit * weights.float()
    return total, z, weight_sum, hit.sum() / weight_sum.clamp_min(1e-8)


def cross_entropy_loss_and_accuracy(source: torch.Tensor, target: torch.Tensor, valid: torch.Tensor | None = None):
    """Mean token cross entropy and accuracy over the ``valid`` positions (no smoothing, no z-loss)."""
    valid = torch.ones_like(target, dtype=torch.float32) if valid is None else valid.float()
    logp = torch.log_softmax(source.float(), -1)
    tok = logp.gather(-1, target.long().clamp_min(0)[..., None])[..., 0] * valid
    n = valid.sum().clamp_min(1e-10)
    loss = -(tok.sum() / n)
    acc = ((source.argmax(-1) == target).float() * valid).sum() / n
    return loss, acc


def fixed_cross_entropy(source: torch.Tensor, target: torch.Tensor, attention_mask: torch.Tensor | None = None,
                        config=None, num_items_in_batch: int | None = None, batch=None, **_):
    """Cross entropy with ``config``'s ignore index, smoothing, z-loss and normalisation
    (easydel/infra/loss_utils.py:1895). Returns a ``LossMetrics``."""
    from .loss_utils import LossConfig, LossMetrics

    cfg = config or LossConfig()
    valid = (target != cfg.ignore_index)
    if attention_mask is not None:
        valid = valid & attention_mask.bool()
    w = valid.float()
    factor = None
    if num_items_in_batch is not None:
        factor = float(num_items_in_batch)
    elif cfg.loss_normalizing_factor is not None and not isinstance(cfg.loss_normalizing_factor, str):
        factor = float(cfg.loss_normalizing_factor)
    total, z, weight_sum, acc = compute_weighted_cross_entropy_and_accuracy(
        source, target.clamp_min(0), w, cfg.label_smoothing, cfg.z_loss, factor)
    if factor is None and cfg.divide_weight_sum:
        total, z = total / weight_sum.clamp_min(1.0), z / weight_sum.clamp_min(1.0)
    return LossMetrics(loss=total, z_loss=z, weight_sum=weight_sum, accuracy=acc)


def sparse_cross_entropy_chunked_vocab(logits: torch.Tensor, labels: torch.Tensor, chunk_size: int = 8192):
    """Per-position ``logsumexp(logits) - logits[label]`` with the log-sum-exp taken over vocabulary chunks (the fp32
    copy of the logits never exists as a whole)."""
    V = logits.shape[-1]
    m = torch.full(logits.shape[:-1], float("-inf"), device=logits.device)
    s = torch.zeros(logits.shape[:-1], device=logits.device)
    for lo in range(0, V, chunk_size):
        c = logits[..., lo:lo + chunk_size].float()
        cm = c.max(-1).values
        new = torch.maximum(m, cm)
        s = s * torch.exp(m - new) + torch.exp(c - new[..., None]).sum(-1)
        m = new
    lse = m + torch.log(s)
    picked = logits.gather(-1, labels.long().clamp(0, V - 1)[..., None])[..., 0].float()
    return lse - picked


def sparse_cross_entropy_chunked_tokens(logits_fn: tp.Callable[[int, int], torch.Tensor], labels: torch.Tensor,
                                        chunk_tokens: int = 2048, ignore_index: int = -100):
    """Sum of token losses and the valid-token count when the logits are produced chunk by chunk:
    ``logits_fn(lo, hi)`` returns the logits of flat token positions ``[lo, hi)``."""
    flat = labels.reshape(-1)
    total = torch.zeros((), device=flat.device)
    count = torch.zeros((), device=flat.device)
    for lo in range(0, flat.numel(), chunk_tokens):
        hi = min(flat.numel(), lo + chunk_tokens)
        lab = flat[lo:hi]
        ok = lab != ignore_index
        lg = logits_fn(lo, hi)
        loss = sparse_cross_entropy_chunked_vocab(lg, lab.clamp_min(0))
        total = total + (loss * ok).sum()
        count = count + ok.sum()
    return total, count


def cross_entropy_blockwise_logits(hidden: torch.Tensor, lm_head_weight: torch.Tensor, labels: torch.Tensor,
                                   block_tokens: int = 2048, ignore_index: int = -100):
    """Mean cross entropy computed from hidden states in token blocks (the ``[tokens, vocab]`` logits exist for one
    block at a time). The CUDA trainers use the fused kernel for this; here it is the reference form."""
    h = hidden.reshape(-1, hidden.shape[-1])
    total, count = sparse_cross_entropy_chunked_tokens(lambda lo, hi: h[lo:hi].float() @ lm_head_weight.float().t(),
                                                       labels, block_tokens, ignore_index)
    return total / count.clamp_min(1.0)


def dynamic_cross_entropy_loss(logits: torch.Tensor, targets: torch.Tensor, weight=None, ignore_index: int | None = -100,
                               reduction: str = "mean", label_smoothing: float = 0.0):
    """Cross entropy with a run-time choice of reduction (``mean`` / ``sum`` / ``none``), class weights, an ignore
    index and smoothing towards the uniform distribution. Returns ``(loss, accuracy)``."""
    V = logits.shape[-1]
    logp = torch.log_softmax(logits.float(), -1)
    t = targets.long()
    ok = torch.ones_like(t, dtype=torch.bool) if ignore_index is None else t != ignore_index
    tc = t.clamp(0, V - 1)
    nll = -logp.gather(-1, tc[..., None])[..., 0]
    if label_smoothing:
        nll = (1.0 - label_smoothing) * nll + label_smoothing * (-logp.mean(-1))
    w = ok.float()
    if weight is not None:
        w = w * weight.float()[tc]
    nll = nll * w
    acc = ((logits.argmax(-1) == t) & ok).float().sum() / ok.float().sum().clamp_min(1.0)
    if reduction == "none":
        return nll, acc
    if reduction == "sum":
        return nll.sum(), acc
    if reduction == "mean":
        return nll.sum() / w.sum().clamp_min(1e-8), acc
    raise ValueError(f"unknown reduction {reduction!r}")


def _sum_weights_per_segment(positions: torch.Tensor, segment_ids: torch.Tensor, weights: torch.Tensor):
    """For every token the total weight of the packed sequence (segment) it belongs to."""
    B, T = segment_ids.shape
    out = torch.zeros_like(weights, dtype=torch.float32)
    for b in range(B):
        seg = segment_ids[b]
        for s in seg.unique():
            m = seg == s
            out[b][m] = weights[b][m].float().sum()
    return out


def get_factor_and_weight(loss_normalizing_factor, batch: tp.Mapping[str, torch.Tensor]):
    """Normalising factor and per-token weights of a batch (easydel/infra/loss_utils.py:1689).

    ``None`` or a number pass through with the batch's ``decoder_loss_weights``; a special factor derives both from
    ``decoder_target_tokens`` (non-zero = real token), ``decoder_loss_weights`` and, for packed batches,
    ``decoder_segment_ids`` / ``decoder_positions``."""
    weights = batch.get("decoder_loss_weights")
    if loss_normalizing_factor is None or isinstance(loss_normalizing_factor, (int, float)):
        return loss_normalizing_factor, weights
    kind = convert_special_loss_normalizing_factor_to_enum(loss_normalizing_factor)
    targets = batch["decoder_target_tokens"]
    real = (targets > 0).float()
    if weights is None:
        weights = real
    weights = weights.float()
    if kind == SLNF.NUM_REAL_TARGET_TOKENS:
        return real.sum(), weights
    if kind == SLNF.NUM_TOTAL_TARGET_TOKENS:
        return float(targets.numel()), weights
    if kind == SLNF.NO_WEIGHT_NUM_REAL_TARGET_TOKENS_DIVIDE_BY_NUM_SEQUENCES:
        return real.sum() / max(1, targets.shape[0]), real
    # AVERAGE_PER_SEQUENCE: every sequence (every segment of a packed row) contributes equally
    seg = batch.get("decoder_segment_ids")
    if seg is None:
        per_seq = weights.sum(-1, keepdim=True)
        n_seq = float(targets.shape[0])
    else:
        per_seq = _sum_weights_per_segment(batch.get("decoder_positions"), seg, weights)
        n_seq = float(sum(int((row[row > 0]).unique().numel()) for row in seg))
    weights = torch.where(per_seq > 0, weights / per_seq.clamp_min(1e-8), torch.zeros_like(weights))
    return n_seq, weights


# ---------------------------------------------------------------------------------------------------- strategies
@dataclasses.dataclass(frozen=True)
class LossForwardPlan:
    """What a loss strategy needs from the forward pass: keyword arguments merged into the model call."""

    forward_kwargs: dict = dataclasses.field(default_factory=dict)


class BaseLossStrategy:
    """Two stages: :meth:`plan_forward` before the model runs, :meth:`compute` on its outputs."""

    __name__ = "BaseLossStrategy"

    def plan_forward(self, *, module, labels, loss_config, batch, loss_kwargs) -> LossForwardPlan:
        return LossForwardPlan()

    def compute(self, *, module, outputs, labels, loss_config, batch, loss_kwargs, loss_scale: float = 1.0):
        raise NotImplementedError


class FunctionalLossStrategy(BaseLossStrategy):
    """Wraps a plain ``loss_fn(logits=..., labels=..., config=..., **kw) -> LossMetrics``."""

    def __init__(self, loss_fn: tp.Callable):
        self.loss_fn = loss_fn
        self.__name__ = getattr(loss_fn, "__name__", type(self).__name__)

    def compute(self, *, module, outputs, labels, loss_config, batch, loss_kwargs, loss_scale: float = 1.0):
        m = self.loss_fn(logits=outputs.logits, labels=labels, config=loss_config,
                         attention_mask=batch.get("attention_mask"), **loss_kwargs)
        if loss_scale != 1.0:
            m.loss = m.loss * loss_scale
        return m


class CausalLMLossStrategy(BaseLossStrategy):
    """Next-token loss that takes hidden states instead of logits: the forward pass is told to skip the LM head and
    the head + cross entropy run fused (CUDA) or in token chunks, so ``[tokens, vocab]`` logits never exist."""

    __name__ = "ForCausalLMLoss"

    def plan_forward(self, *, module, labels, loss_config, batch, loss_kwargs) -> LossForwardPlan:
        if labels is None or not hasattr(module, "lm_head_weight"):
            return LossForwardPlan()
        return LossForwardPlan({"apply_lm_head": False})

    def compute(self, *, module, outputs, labels, loss_config, batch, loss_kwargs, loss_scale: float = 1.0):
        from .loss_utils import ForCausalLMLoss, causal_lm_loss_from_hidden

        if getattr(outputs, "logits", None) is not None:
            m = ForCausalLMLoss(outputs.logits, labels, batch.get("attention_mask"), loss_config, **loss_kwargs)
            m.loss = m.loss * loss_scale
            return m
        return causal_lm_loss_from_hidden(outputs.last_hidden_state, module.lm_head_weight(), labels, loss_config,
                                          lm_head_bias=module.lm_head_bias(),
                                          chunk_size=getattr(module.config, "lmhead_chunksize", None),
                                          loss_scale=loss_scale, **loss_kwargs)


def resolve_loss_strategy(loss_fn) -> BaseLossStrategy:
    """A strategy for a task-loss function (or a strategy, passed through)."""
    if isinstance(loss_fn, BaseLossStrategy):
        return loss_fn
    if getattr(loss_fn, "__name__", "") == "ForCausalLMLoss":
        return CausalLMLossStrategy()
    return FunctionalLossStrategy(loss_fn)
