"""Token / sequence log-probabilities without materialising ``[tokens, vocab]`` logits.

The preference and RL trainers need ``log pi(y_t | y_<t)`` for given tokens, sometimes with the
policy entropy. The reference computes them from chunked logits (easydel/trainers/_logprob_utils.py and
direct_preference_optimization_trainer/_fn.py:63); here the backbone runs once, and the LM head is folded
into the fused head+log-prob kernel (``ops.functional.linear_token_logprob``), chunked over tokens.
"""

from __future__ import annotations

import torch

from ..ops import functional as F


def _head(model):
    w = model.lm_head_weight() if hasattr(model, "lm_head_weight") else None
    b = model.lm_head_bias() if hasattr(model, "lm_head_bias") else None
    return w, b


def token_logprobs(model, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None,
                   loss_mask: torch.Tensor | None = None, *, temperature: float = 1.0, want_entropy: bool = False,
                   chunk_size: int = 2048, **model_kwargs):
    """Returns ``(logps [B, T-1], mask [B, T-1] float, entropy or None, model_output)``.

    ``logps[b, t]`` is the log-probability of ``input_ids[b, t+1]``; positions outside ``loss_mask`` (which is
    aligned with ``input_ids``) or outside ``attention_mask`` are zero.
    """
    mask = torch.ones_like(input_ids, dtype=torch.bool) if loss_mask is None else loss_mask.bool()
    if attention_mask is not None:
        mask = mask & attention_mask.bool()
    mask = mask[:, 1:]
    labels = input_ids[:, 1:].masked_fill(~mask, -100)
    w, b = _head(model)
    spec = getattr(model, "spec", None)
    direct = w is not None and not (spec is not None and spec.logit_softcap)
    if direct:
        sp_kw = {}
        if getattr(getattr(model, "model", None), "sp_capable", False) and "sequence_parallel" not in model_kwargs:
            sp_kw["sequence_parallel"] = True   # tensor-parallel dense stacks keep the token rows sharded
        out = model(input_ids=input_ids, attention_mask=attention_mask, apply_lm_head=False, **sp_kw, **model_kwargs)
        sp = getattr(getattr(model, "model", None), "sp", None)
        if sp is not None and sp.active:
            lp, ent = _token_logprobs_row_sharded(model, sp, out.last_hidden_state, labels, w, b, spec, temperature,
                                                  chunk_size, want_entropy)
        else:
            h = out.last_hidden_state[:, :-1]
            if spec is not None and spec.logit_scale is not None:
                h = h * spec.logit_scale
            lp, ent = F.linear_token_logprob(h, w, labels, bias=b, temperature=temperature, chunk_size=chunk_size,
                                             want_entropy=want_entropy)
    else:
        out = model(input_ids=input_ids, attention_mask=attention_mask, **model_kwargs)
        logits = out.logits[:, :-1].float() / temperature
        lsm = torch.log_softmax(logits, -1)
        lp = lsm.gather(-1, labels.clamp_min(0)[..., None])[..., 0]
        ent = -(lsm.exp() * lsm).sum(-1) if want_entropy else None
    m = mask.to(lp.dtype)
    lp = lp * m
    if ent is not None:
        ent = ent * m
    return lp, m, ent, out


def _token_logprobs_row_sharded(model, sp, h_shard, labels, w, b, spec, temperature, chunk_size, want_entropy):
    """Log-probabilities when the backbone returned this rank's rows of the flattened token axis (sequence-parallel
    tensor parallelism). Each rank scores its rows; the rows of all ranks are then summed into the full
    ``[B, T-1]`` table on every rank. What follows is the same computation on every rank, so each rank
    back-propagates only through its own rows and parameter gradients are partial sums over the group
    (``sp_partial_grads``: completed before the optimizer update)."""
    from ..parallel import tp as tpar

    B, T = sp.batch, sp.seq
    full_labels = torch.full((B, T), -100, dtype=labels.dtype, device=labels.device)
    full_labels[:, :-1] = labels
    lab = tpar.shard_rows(sp, full_labels).reshape(-1)
    h = h_shard.reshape(-1, h_shard.shape[-1])
    if spec is not None and spec.logit_scale is not None:
        h = h * spec.logit_scale
    lp, ent = F.linear_token_logprob(h[None], w, lab[None], bias=b, temperature=temperature, chunk_size=chunk_size,
                                     want_entropy=want_entropy)
    n, r = sp.rows_local, sp.rank

    def spread(v):
        v = torch.nn.functional.pad(v.reshape(-1), (r * n, (sp.world - 1 - r) * n))
        return tpar.sum_value_over_group(v, sp.group).view(B, T)[:, :-1]

    if torch.is_grad_enabled() and h.requires_grad:
        model.sp_partial_grads = True
    return spread(lp), (spread(ent) if ent is not None else None)


def sequence_logprobs(model, input_ids, attention_mask=None, loss_mask=None, *, average: bool = False, **kw):
    """Sum (or mean) of the token log-probabilities over ``loss_mask``: ``[B]``."""
    lp, m, _, out = token_logprobs(model, input_ids, attention_mask, loss_mask, **kw)
    s = lp.sum(-1)
    if average:
        s = s / m.sum(-1).clamp_min(1.0)
    return s, m.sum(-1), out


def masked_mean(x: torch.Tensor, mask: torch.Tensor, dim=None) -> torch.Tensor:
    if dim is None:
        return (x * mask).sum() / mask.sum().clamp_min(1.0)
    return (x * mask).sum(dim) / mask.sum(dim).clamp_min(1.0)


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    return torch.log_softmax(logits.float(), -1).gather(-1, index[..., None])[..., 0]
