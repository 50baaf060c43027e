"""RoBERTa: bidirectional post-LayerNorm encoder with masked-LM, sequence- and token-classification heads
(easydel/modules/roberta).

Encoder layer: ``x = LN(x + attn(x)); x = LN(x + mlp(x))`` with full (non-causal) attention; padding is kept out
through segment ids (0 = padding). Embeddings: word + learned position (offset by ``pad_token_id + 1``, counted over
non-padding tokens) + token type, then LayerNorm. Weight names are mapped to and from the Hugging Face checkpoint
names by the renaming table at the bottom.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.loss_utils import LossConfig, LossMetrics
from ...infra.modeling_outputs import BaseModelOutput, CausalLMOutput, SequenceClassifierOutput
from ...layers.attention import Attention
from ...layers.embeddings import Embed
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import PlainMLP
from ...layers.norms import LayerNorm
from .._base.families import _Renamer


@register_config("roberta")
class RobertaConfig(EasyDeLBaseConfig):
    model_type = "roberta"
    hf_config_keys = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                      "hidden_act", "hidden_dropout_prob", "attention_probs_dropout_prob", "max_position_embeddings",
                      "type_vocab_size", "initializer_range", "layer_norm_eps", "classifier_dropout")

    def __init__(self, vocab_size=50265, hidden_size=768, num_hidden_layers=12, num_attention_heads=12,
                 intermediate_size=3072, hidden_act="gelu", hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                 max_position_embeddings=514, type_vocab_size=1, initializer_range=0.02, layer_norm_eps=1e-5,
                 pad_token_id=1, bos_token_id=0, eos_token_id=2, classifier_dropout=None, **kw):
        self.vocab_size, self.hidden_size, self.num_hidden_layers = vocab_size, hidden_size, num_hidden_layers
        self.num_attention_heads, self.intermediate_size, self.hidden_act = num_attention_heads, intermediate_size, \
            hidden_act
        self.hidden_dropout_prob, self.attention_probs_dropout_prob = hidden_dropout_prob, attention_probs_dropout_prob
        self.max_position_embeddings, self.type_vocab_size = max_position_embeddings, type_vocab_size
        self.initializer_range, self.layer_norm_eps, self.classifier_dropout = initializer_range, layer_norm_eps, \
            classifier_dropout
        super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id, **kw)


class RobertaLayer(nn.Module):
    def __init__(self, c: RobertaConfig, idx: int, dtype):
        super().__init__()
        hd = c.hidden_size // c.num_attention_heads
        self.self_attn = Attention(c.hidden_size, c.num_attention_heads, c.num_attention_heads, hd, layer_idx=idx,
                                   bias=True, o_bias=True, rope=None, causal=False, dtype=dtype,
                                   init_std=c.initializer_range)
        self.attention_norm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)
        self.mlp = PlainMLP(c.hidden_size, c.intermediate_size, c.hidden_act, True, dtype, c.initializer_range)
        self.output_norm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)

    def forward(self, x, positions, segment_ids):
        x = self.attention_norm(x + self.self_attn(x, positions, segment_ids=segment_ids))
        return self.output_norm(x + self.mlp(x))


class _Embeddings(nn.Module):
    def __init__(self, c: RobertaConfig, dtype):
        super().__init__()
        self.pad = c.pad_token_id
        self.word_embeddings = Embed(c.vocab_size, c.hidden_size, dtype, c.initializer_range)
        self.position_embeddings = Embed(c.max_position_embeddings, c.hidden_size, dtype, c.initializer_range)
        self.token_type_embeddings = Embed(c.type_vocab_size, c.hidden_size, dtype, c.initializer_range)
        self.LayerNorm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)

    def forward(self, input_ids, token_type_ids=None, position_ids=None):
        if position_ids is None:
            mask = (input_ids != self.pad).long()
            position_ids = mask.cumsum(1) * mask + self.pad
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(input_ids)
        x = self.word_embeddings(input_ids) + self.position_embeddings(position_ids) + \
            self.token_type_embeddings(token_type_ids)
        return self.LayerNorm(x)


_RULES = [("roberta.embeddings.", "model.embeddings."), ("roberta.encoder.layer.", "model.layers."),
          (".attention.self.query.", ".self_attn.q_proj."), (".attention.self.key.", ".self_attn.k_proj."),
          (".attention.self.value.", ".self_attn.v_proj."), (".attention.output.dense.", ".self_attn.o_proj."),
          (".attention.output.LayerNorm.", ".attention_norm."), (".intermediate.dense.", ".mlp.fc1."),
          (".output.dense.", ".mlp.fc2."), (".output.LayerNorm.", ".output_norm.")]
_REN = _Renamer(_RULES)


class _RobertaBase(EasyDeLBaseModule):
    hf_keeps_fused = ()

    def hf_rename_in(self, sd):
        sd = {k: v for k, v in sd.items() if not k.endswith("position_ids")}
        if not any(k.startswith("roberta.") for k in sd):      # bare encoder checkpoints carry no prefix
            sd = {("roberta." + k if k.split(".")[0] in ("embeddings", "encoder") else k): v for k, v in sd.items()}
        return _REN.to_internal(self, sd)

    def hf_rename_out(self, sd):
        return _REN.to_hf(self, sd)


@register_module(TaskType.BASE_MODULE, config=RobertaConfig, model_type="roberta",
                 layernorm_names=["LayerNorm", "attention_norm", "output_norm", "layer_norm"])
class RobertaModel(_RobertaBase):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.embeddings = _Embeddings(config, pd)
        self.layers = nn.ModuleList([RobertaLayer(config, i, pd) for i in range(config.num_hidden_layers)])

    def get_input_embeddings(self):
        return self.embeddings.word_embeddings

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, position_ids=None,
                output_hidden_states=False, **_):
        x = self.embeddings(input_ids, token_type_ids, position_ids)
        if x.dtype != self.dtype:
            x = x.to(self.dtype)
        seg = None
        if attention_mask is not None and not bool(attention_mask.all()):
            seg = attention_mask.to(torch.int32)
        B, T = input_ids.shape
        pos = torch.arange(T, device=x.device)[None].expand(B, T)
        hs = [] if output_hidden_states else None
        for layer in self.layers:
            if hs is not None:
                hs.append(x)
            x = layer(x, pos, seg)
        if hs is not None:
            hs.append(x)
        return BaseModelOutput(last_hidden_state=x, hidden_states=tuple(hs) if hs else None)


class _LMHead(nn.Module):
    def __init__(self, c, dtype):
        super().__init__()
        self.dense = ColumnParallelLinear(c.hidden_size, c.hidden_size, bias=True, dtype=dtype,
                                          init_std=c.initializer_range)
        self.layer_norm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)
        self.bias = nn.Parameter(torch.zeros(c.vocab_size, dtype=dtype))

    def forward(self, h, embed_weight):
        from ...ops import functional as F

        x = self.layer_norm(torch.nn.functional.gelu(self.dense(h)))
        return F.linear(x, embed_weight, self.bias)


@register_module(TaskType.CAUSAL_LM, config=RobertaConfig, model_type="roberta")
class RobertaForMaskedLM(_RobertaBase):
    """Registered under the language-modelling task; the loss is the masked-LM loss (labels -100 outside masks)."""

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.model = RobertaModel(config, dtype, param_dtype, precision, rngs)
        self.lm_head = _LMHead(config, self.param_dtype)

    def hf_rename_in(self, sd):
        sd = {k: v for k, v in sd.items() if k not in ("lm_head.decoder.weight", "lm_head.decoder.bias")}
        return super().hf_rename_in(sd)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, position_ids=None, **kw):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, token_type_ids=token_type_ids,
                         position_ids=position_ids, **kw)
        logits = self.lm_head(out.last_hidden_state, self.model.embeddings.word_embeddings.weight)
        return CausalLMOutput(logits=logits, last_hidden_state=out.last_hidden_state, hidden_states=out.hidden_states)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        out = self(**call)
        lg = out.logits.float()
        loss = torch.nn.functional.cross_entropy(lg.view(-1, lg.shape[-1]), labels.reshape(-1),
                                                 ignore_index=loss_config.ignore_index)
        return out, LossMetrics(loss=loss * loss_scale)


class _ClassificationHead(nn.Module):
    def __init__(self, c, dtype, num_labels):
        super().__init__()
        self.dense = ColumnParallelLinear(c.hidden_size, c.hidden_size, bias=True, dtype=dtype,
                                          init_std=c.initializer_range)
        self.out_proj = ColumnParallelLinear(c.hidden_size, num_labels, bias=True, dtype=dtype,
                                             init_std=c.initializer_range)

    def forward(self, h):
        return self.out_proj(torch.tanh(self.dense(h[:, 0])))


@register_module(TaskType.SEQUENCE_CLASSIFICATION, config=RobertaConfig, model_type="roberta")
class RobertaForSequenceClassification(_RobertaBase):
    loss_type = "ForSequenceClassification"

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.num_labels = getattr(config, "num_labels", 2)
        self.model = RobertaModel(config, dtype, param_dtype, precision, rngs)
        self.classifier = _ClassificationHead(config, self.param_dtype, self.num_labels)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, position_ids=None, **kw):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, token_type_ids=token_type_ids,
                         position_ids=position_ids)
        return SequenceClassifierOutput(logits=self.classifier(out.last_hidden_state),
                                        hidden_states=out.hidden_states)

    def _compute_task_loss(self, labels, loss_config, loss_scale, call, loss_kwargs):
        from ...infra.loss_utils import ForSequenceClassificationLoss

        out = self(**call)
        m = ForSequenceClassificationLoss(out.logits, labels, loss_config)
        m.loss = m.loss * loss_scale
        return out, m


class RobertaForTokenClassification(_RobertaBase):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.num_labels = getattr(config, "num_labels", 2)
        self.model = RobertaModel(config, dtype, param_dtype, precision, rngs)
        self.classifier = ColumnParallelLinear(config.hidden_size, self.num_labels, bias=True, dtype=self.param_dtype,
                                               init_std=config.initializer_range)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, position_ids=None, **kw):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, token_type_ids=token_type_ids,
                         position_ids=position_ids)
        return SequenceClassifierOutput(logits=self.classifier(out.last_hidden_state),
                                        hidden_states=out.hidden_states)
