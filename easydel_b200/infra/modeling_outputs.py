"""Typed model outputs (easydel/infra/modeling_outputs.py:136-1726).

A single ``ModelOutput`` base gives attribute, key and index access; the concrete classes
only declare their fields.
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass, fields

import torch


@dataclass
class ModelOutput:
    def __getitem__(self, k):
        if isinstance(k, str):
            return getattr(self, k)
        return self.to_tuple()[k]

    def keys(self):
        return [f.name for f in fields(self) if getattr(self, f.name) is not None]

    def items(self):
        return [(k, getattr(self, k)) for k in self.keys()]

    def get(self, k, default=None):
        v = getattr(self, k, None)
        return default if v is None else v

    def to_tuple(self):
        return tuple(getattr(self, k) for k in self.keys())

    def __contains__(self, k):
        return k in self.keys()

    def replace(self, **kw):
        import dataclasses

        return dataclasses.replace(self, **kw)


@dataclass
class BaseModelOutput(ModelOutput):
    last_hidden_state: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None
    past_key_values: tp.Any = None


BaseModelOutputWithPast = BaseModelOutput


@dataclass
class MoeModelOutput(BaseModelOutput):
    router_logits: tuple | None = None
    all_router_losses: tuple | None = None


@dataclass
class CausalLMOutput(ModelOutput):
    logits: torch.Tensor | None = None
    loss: torch.Tensor | None = None
    last_hidden_state: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None
    past_key_values: tp.Any = None


CausalLMOutputWithPast = CausalLMOutput


@dataclass
class MoeCausalLMOutput(CausalLMOutput):
    aux_loss: torch.Tensor | None = None
    router_logits: tuple | None = None
    all_router_losses: tuple | None = None


@dataclass
class SequenceClassifierOutput(ModelOutput):
    logits: torch.Tensor | None = None
    loss: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None
    past_key_values: tp.Any = None
    aux_loss: torch.Tensor | None = None


@dataclass
class TokenClassifierOutput(SequenceClassifierOutput):
    pass


@dataclass
class QuestionAnsweringModelOutput(ModelOutput):
    start_logits: torch.Tensor | None = None
    end_logits: torch.Tensor | None = None
    loss: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None


@dataclass
class EmbeddingOutput(ModelOutput):
    embeddings: torch.Tensor | None = None
    last_hidden_state: torch.Tensor | None = None
    loss: torch.Tensor | None = None


@dataclass
class BaseModelOutputWithPooling(BaseModelOutput):
    pooler_output: torch.Tensor | None = None


@dataclass
class ImageClassifierOutput(SequenceClassifierOutput):
    pass


@dataclass
class Seq2SeqModelOutput(ModelOutput):
    last_hidden_state: torch.Tensor | None = None
    past_key_values: tp.Any = None
    decoder_hidden_states: tuple | None = None
    decoder_attentions: tuple | None = None
    cross_attentions: tuple | None = None
    encoder_last_hidden_state: torch.Tensor | None = None
    encoder_hidden_states: tuple | None = None
    encoder_attentions: tuple | None = None


@dataclass
class Seq2SeqLMOutput(Seq2SeqModelOutput):
    logits: torch.Tensor | None = None
    loss: torch.Tensor | None = None


@dataclass
class VLMCausalLMOutput(CausalLMOutput):
    image_hidden_states: torch.Tensor | None = None
    rope_deltas: torch.Tensor | None = None
    aux_loss: torch.Tensor | None = None
    router_logits: tuple | None = None


@dataclass
class CLIPOutput(ModelOutput):
    loss: torch.Tensor | None = None
    logits_per_image: torch.Tensor | None = None
    logits_per_text: torch.Tensor | None = None
    text_embeds: torch.Tensor | None = None
    image_embeds: torch.Tensor | None = None
    text_model_output: tp.Any = None
    vision_model_output: tp.Any = None


@dataclass
class GreedySearchOutput(ModelOutput):
    sequences: torch.Tensor | None = None


@dataclass
class SampleOutput(ModelOutput):
    sequences: torch.Tensor | None = None


@dataclass
class BeamSearchOutput(ModelOutput):
    sequences: torch.Tensor | None = None
    scores: torch.Tensor | None = None


# ---- the remaining output types of the reference's module (same field names; only the fields differ) ----------------
@dataclass
class EmbeddingInfo(ModelOutput):
    """What ``get_embedding_info`` reports about a model's embedding tables."""

    vocab_size: int | None = None
    hidden_size: int | None = None
    tie_word_embeddings: bool | None = None
    embedding_names: tuple | None = None


@dataclass
class AttentionLayerOutput(ModelOutput):
    attention_output: torch.Tensor | None = None
    attention_weight: torch.Tensor | None = None
    cache_view: tp.Any = None


@dataclass
class EncoderLayerOutput(ModelOutput):
    hidden_states: torch.Tensor | None = None
    residual_states: torch.Tensor | None = None
    attention_weight: torch.Tensor | None = None


@dataclass
class DecoderLayerOutput(ModelOutput):
    hidden_states: torch.Tensor | None = None
    residual_states: torch.Tensor | None = None
    attention_weight: torch.Tensor | None = None
    cross_attention_weight: torch.Tensor | None = None
    router_logits: torch.Tensor | None = None
    gate_loss: torch.Tensor | None = None
    cache_view: tp.Any = None


@dataclass
class BaseModelOutputWithNoAttention(ModelOutput):
    last_hidden_state: torch.Tensor | None = None
    hidden_states: tuple | None = None


@dataclass
class BaseModelOutputWithPoolingAndNoAttention(BaseModelOutputWithNoAttention):
    pooler_output: torch.Tensor | None = None


@dataclass
class ImageClassifierOutputWithNoAttention(ModelOutput):
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    hidden_states: tuple | None = None


@dataclass
class BaseModelOutputWithPoolingAndCrossAttentions(BaseModelOutput):
    pooler_output: torch.Tensor | None = None
    cross_attentions: tuple | None = None


@dataclass
class BaseModelOutputWithPastAndCrossAttentions(BaseModelOutput):
    cross_attentions: tuple | None = None


@dataclass
class CausalLMOutputWithCrossAttentions(ModelOutput):
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    last_hidden_state: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None
    cross_attentions: tuple | None = None
    past_key_values: tp.Any = None


@dataclass
class MaskedLMOutput(ModelOutput):
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    last_hidden_state: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None


@dataclass
class NextSentencePredictorOutput(ModelOutput):
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None


@dataclass
class Seq2SeqSequenceClassifierOutput(ModelOutput):
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    past_key_values: tp.Any = None
    decoder_hidden_states: tuple | None = None
    decoder_attentions: tuple | None = None
    cross_attentions: tuple | None = None
    encoder_last_hidden_state: torch.Tensor | None = None
    encoder_hidden_states: tuple | None = None
    encoder_attentions: tuple | None = None


@dataclass
class MultipleChoiceModelOutput(ModelOutput):
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None


@dataclass
class Seq2SeqQuestionAnsweringModelOutput(ModelOutput):
    loss: torch.Tensor | None = None
    start_logits: torch.Tensor | None = None
    end_logits: torch.Tensor | None = None
    past_key_values: tp.Any = None
    decoder_hidden_states: tuple | None = None
    decoder_attentions: tuple | None = None
    cross_attentions: tuple | None = None
    encoder_last_hidden_state: torch.Tensor | None = None
    encoder_hidden_states: tuple | None = None
    encoder_attentions: tuple | None = None


@dataclass
class MambaOutput(ModelOutput):
    last_hidden_state: torch.Tensor | None = None
    cache_params: tp.Any = None
    hidden_states: tuple | None = None


@dataclass
class MambaCausalLMOutput(ModelOutput):
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    cache_params: tp.Any = None
    last_hidden_state: torch.Tensor | None = None
    hidden_states: tuple | None = None


@dataclass
class CLIPTextModelOutput(ModelOutput):
    text_embeds: torch.Tensor | None = None
    last_hidden_state: torch.Tensor | None = None
    hidden_states: tuple | None = None
    attentions: tuple | None = None
