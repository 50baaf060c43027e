"""Llama family (easydel/modules/llama/modeling_llama.py:48-613)."""

from __future__ import annotations

from ...infra.factory import TaskType, register_module
from .._base.decoder import ArchSpec, DecoderForCausalLM, DecoderForSequenceClassification, DecoderModel
from .configuration import LlamaConfig


def llama_spec(c) -> ArchSpec:
    rope_scaling = getattr(c, "rope_scaling", None)
    rope_params = getattr(c, "rope_parameters", None)
    theta = getattr(c, "rope_theta", None)
    if rope_params and isinstance(rope_params, dict):
        theta = theta or rope_params.get("rope_theta")
        if rope_scaling is None and rope_params.get("rope_type", "default") != "default":
            rope_scaling = {k: v for k, v in rope_params.items() if k != "rope_theta"}
    return ArchSpec(
        hidden_size=c.hidden_size, num_layers=c.num_hidden_layers, num_heads=c.num_attention_heads,
        num_kv_heads=c.num_key_value_heads, head_dim=c.head_dim, intermediate_size=c.intermediate_size,
        vocab_size=c.vocab_size, max_position=c.max_position_embeddings, norm="rms", norm_eps=c.rms_norm_eps,
        act=c.hidden_act, mlp="gated", mlp_bias=getattr(c, "mlp_bias", False),
        attn_bias=getattr(c, "attention_bias", False), o_bias=getattr(c, "attention_bias", False),
        rope=dict(rotary_dim=c.head_dim, max_position=c.max_position_embeddings, base=theta or 10000.0,
                  is_neox_style=True, rope_scaling=rope_scaling),
        tie_embeddings=getattr(c, "tie_word_embeddings", False), init_std=c.initializer_range)


@register_module(TaskType.BASE_MODULE, config=LlamaConfig, model_type="llama")
class LlamaModel(DecoderModel):
    spec_fn = staticmethod(llama_spec)


@register_module(TaskType.CAUSAL_LM, config=LlamaConfig, model_type="llama")
class LlamaForCausalLM(DecoderForCausalLM):
    backbone_cls = LlamaModel


@register_module(TaskType.SEQUENCE_CLASSIFICATION, config=LlamaConfig, model_type="llama")
class LlamaForSequenceClassification(DecoderForSequenceClassification):
    backbone_cls = LlamaModel
