"""Contrastive embedding trainer (easydel/trainers/embedding_trainer).

Rows carry a query and a positive passage (optionally hard negatives); the loss is InfoNCE over in-batch
negatives on pooled, L2-normalised hidden states, optionally at several Matryoshka dimensions.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as tF

from ..infra.loss_utils import LossMetrics
from .base_trainer import Trainer
from .training_configurations import TrainingArguments, register_trainer, register_trainer_arguments
from .utils import pad_to_length


@register_trainer_arguments("embedding")
@dataclass
class EmbeddingConfig(TrainingArguments):
    trainer_prefix: str | None = "embeddingtrainer"
    pooling: str = "last"                    # last | mean | cls
    temperature: float = 0.05
    normalize: bool = True
    matryoshka_dims: tuple[int, ...] | None = None
    symmetric: bool = False                  # add the passage->query direction
    gather_negatives_across_ranks: bool = True


class EmbeddingCollator:
    def __init__(self, pad_token_id: int = 0, max_length: int | None = None):
        self.pad, self.max_length = pad_token_id, max_length

    def __call__(self, feats):
        out = {}
        for key in ("query", "positive", "negative"):
            if f"{key}_input_ids" not in feats[0]:
                continue
            rows = [torch.as_tensor(f[f"{key}_input_ids"], dtype=torch.long)[: self.max_length] for f in feats]
            L = max(r.shape[0] for r in rows)
            out[f"{key}_input_ids"] = torch.stack([pad_to_length(r, L, self.pad) for r in rows])
            out[f"{key}_attention_mask"] = torch.stack([pad_to_length(torch.ones_like(r), L, 0) for r in rows])
        return out


def pool_hidden(h: torch.Tensor, mask: torch.Tensor, how: str) -> torch.Tensor:
    if how == "mean":
        m = mask[..., None].to(h.dtype)
        return (h * m).sum(1) / m.sum(1).clamp_min(1)
    if how == "cls":
        return h[:, 0]
    last = (mask.long() * torch.arange(mask.shape[1], device=mask.device)[None]).argmax(1)
    return h[torch.arange(h.shape[0], device=h.device), last]


def info_nce(q: torch.Tensor, p: torch.Tensor, neg: torch.Tensor | None, temperature: float, symmetric: bool):
    cands = p if neg is None else torch.cat([p, neg], 0)
    logits = q @ cands.t() / temperature
    target = torch.arange(q.shape[0], device=q.device)
    loss = tF.cross_entropy(logits, target)
    if symmetric:
        loss = 0.5 * (loss + tF.cross_entropy(p @ q.t() / temperature, target))
    return loss, (logits.argmax(-1) == target).float().mean()


@register_trainer("embedding")
class EmbeddingTrainer(Trainer):
    trainer_type = "embedding"
    arguments_class = EmbeddingConfig

    def __init__(self, arguments=None, model=None, processing_class=None, train_dataset=None, eval_dataset=None,
                 data_collator=None, **kw):
        arguments = arguments or EmbeddingConfig()
        pad = getattr(processing_class, "pad_token_id", None) or 0
        super().__init__(arguments=arguments, model=model, dataset_train=kw.pop("dataset_train", train_dataset),
                         dataset_eval=kw.pop("dataset_eval", eval_dataset),
                         data_collator=data_collator or EmbeddingCollator(pad, arguments.max_length),
                         processing_class=processing_class, **kw)

    def encode(self, model, ids, mask):
        out = model(input_ids=ids, attention_mask=mask, apply_lm_head=False) if hasattr(model, "lm_head_weight") \
            else model(input_ids=ids, attention_mask=mask)
        h = out.last_hidden_state.float()
        return pool_hidden(h, mask, self.arguments.pooling)

    def compute_step_loss(self, model, batch, loss_scale, is_train):
        a = self.arguments
        q = self.encode(model, batch["query_input_ids"], batch["query_attention_mask"])
        p = self.encode(model, batch["positive_input_ids"], batch["positive_attention_mask"])
        n = self.encode(model, batch["negative_input_ids"], batch["negative_attention_mask"]) \
            if "negative_input_ids" in batch else None
        dims = a.matryoshka_dims or (q.shape[-1],)
        total, acc = 0.0, None
        for d in dims:
            qq, pp, nn_ = q[:, :d], p[:, :d], (n[:, :d] if n is not None else None)
            if a.normalize:
                qq, pp = tF.normalize(qq, dim=-1), tF.normalize(pp, dim=-1)
                nn_ = tF.normalize(nn_, dim=-1) if nn_ is not None else None
            l, acc_d = info_nce(qq, pp, nn_, a.temperature, a.symmetric)
            total = total + l
            acc = acc_d if acc is None else acc
        return LossMetrics(loss=total / len(dims) * loss_scale, accuracy=acc.detach())
