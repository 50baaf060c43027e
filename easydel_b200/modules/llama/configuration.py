"""Llama configuration (easydel/modules/llama/llama_configuration.py:98-184)."""

from __future__ import annotations

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import register_config


@register_config("llama")
class LlamaConfig(EasyDeLBaseConfig):
    model_type = "llama"

    def __init__(self, vocab_size: int = 32000, hidden_size: int = 4096, intermediate_size: int = 11008,
                 num_hidden_layers: int = 32, num_attention_heads: int = 32, num_key_value_heads: int | None = None,
                 head_dim: int | None = None, hidden_act: str = "silu", max_position_embeddings: int = 2048,
                 initializer_range: float = 0.02, rms_norm_eps: float = 1e-6, use_cache: bool = True,
                 pad_token_id: int | None = None, bos_token_id: int = 1, eos_token_id: int = 2,
                 tie_word_embeddings: bool = False, rope_theta: float = 10000.0, rope_scaling: dict | None = None,
                 attention_bias: bool = False, attention_dropout: float = 0.0, mlp_bias: bool = False, **kwargs):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_hidden_layers = num_hidden_layers
        self.num_attention_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads if num_key_value_heads is not None else num_attention_heads
        self.head_dim = head_dim if head_dim is not None else hidden_size // num_attention_heads
        self.hidden_act = hidden_act
        self.max_position_embeddings = max_position_embeddings
        self.initializer_range = initializer_range
        self.rms_norm_eps = rms_norm_eps
        self.use_cache = use_cache
        self.rope_theta = rope_theta
        self.rope_scaling = rope_scaling
        self.attention_bias = attention_bias
        self.attention_dropout = attention_dropout
        self.mlp_bias = mlp_bias
        super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                         tie_word_embeddings=tie_word_embeddings, **kwargs)
