"""Decoder-only text families defined through the spec table (see ``_base/families.py``).

Each block cites the reference directory it covers (easydel/modules/<family>/). Config defaults
follow the Hugging Face configs of the same ``model_type`` so that ``config.json`` files load
unchanged.
"""

from __future__ import annotations

import math
import re

import torch

from ._base.decoder import ArchSpec, MoESpec
from ._base.families import base_spec, define_family, moe_spec, rope_args

_LLAMA_DEFAULTS = dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=None, head_dim=None, hidden_act="silu",
                       max_position_embeddings=4096, initializer_range=0.02, rms_norm_eps=1e-6, use_cache=True,
                       rope_theta=10000.0, rope_scaling=None, attention_bias=False, attention_dropout=0.0,
                       mlp_bias=False, tie_word_embeddings=False)
EXPORTS: dict[str, type] = {}


def _d(**kw):
    d = dict(_LLAMA_DEFAULTS)
    d.update(kw)
    return d


def _layer_types(c, n):
    lt = getattr(c, "layer_types", None)
    if lt:
        return tuple("sliding" if "sliding" in t else "full" for t in lt)
    return None


# ---- mistral (easydel/modules/mistral) ------------------------------------------------------
EXPORTS.update(define_family("mistral", _d(sliding_window=4096, rms_norm_eps=1e-6, max_position_embeddings=32768),
                             lambda c: base_spec(c, sliding_window=getattr(c, "sliding_window", None))))

# ---- qwen2 (easydel/modules/qwen2): biased q/k/v ----------------------------------------------
EXPORTS.update(define_family(
    "qwen2", _d(vocab_size=151936, intermediate_size=22016, max_position_embeddings=32768, use_sliding_window=False,
                sliding_window=4096, max_window_layers=28, layer_types=None),
    lambda c: base_spec(c, attn_bias=True, o_bias=False,
                        sliding_window=c.sliding_window if getattr(c, "use_sliding_window", False) else None)))

# ---- qwen3 (easydel/modules/qwen3): per-head QK RMSNorm ---------------------------------------
EXPORTS.update(define_family(
    "qwen3", _d(vocab_size=151936, intermediate_size=22016, head_dim=128, max_position_embeddings=32768,
                use_sliding_window=False, sliding_window=None, layer_types=None),
    lambda c: base_spec(c, qk_norm="rms_head")))

# ---- seed_oss / smollm3 / granite -----------------------------------------------------------
EXPORTS.update(define_family("seed_oss", _d(attention_bias=True, attention_out_bias=False, head_dim=128),
                             lambda c: base_spec(c, attn_bias=c.attention_bias,
                                                 o_bias=getattr(c, "attention_out_bias", False))))


def _smollm3_spec(c):
    n = c.num_hidden_layers
    nope = getattr(c, "no_rope_layers", None)
    if nope is None:
        interval = getattr(c, "no_rope_layer_interval", 4)
        nope = [int((i + 1) % interval != 0) for i in range(n)]
    lt = tuple("full" if nope[i] else "nope" for i in range(n))
    return base_spec(c, layer_types=lt)


EXPORTS.update(define_family("smollm3", _d(no_rope_layers=None, no_rope_layer_interval=4, use_sliding_window=False,
                                           sliding_window=None, layer_types=None), _smollm3_spec,
                             class_prefix="SmolLM3"))
EXPORTS.update(define_family(
    "granite", _d(embedding_multiplier=1.0, logits_scaling=1.0, residual_multiplier=1.0, attention_multiplier=1.0),
    lambda c: base_spec(c, embedding_multiplier=c.embedding_multiplier, residual_multiplier=c.residual_multiplier,
                        attn_scale=c.attention_multiplier, logit_scale=1.0 / c.logits_scaling)))

# ---- gemma family (easydel/modules/gemma, gemma2, gemma3) --------------------------------------
_GEMMA = _d(vocab_size=256000, hidden_size=3072, intermediate_size=24576, num_hidden_layers=28,
            num_attention_heads=16, num_key_value_heads=16, head_dim=256, hidden_act="gelu_pytorch_tanh",
            hidden_activation="gelu_pytorch_tanh", max_position_embeddings=8192, tie_word_embeddings=True)


def _gemma_act(c):
    return getattr(c, "hidden_activation", None) or "gelu_pytorch_tanh"


EXPORTS.update(define_family(
    "gemma", _GEMMA,
    lambda c: base_spec(c, norm_offset=1.0, act=_gemma_act(c), embed_scale=math.sqrt(c.hidden_size),
                        tie_embeddings=True)))


def _gemma2_spec(c):
    n = c.num_hidden_layers
    lt = _layer_types(c, n) or tuple("sliding" if i % 2 == 0 else "full" for i in range(n))
    return base_spec(c, norm_offset=1.0, act=_gemma_act(c), embed_scale=math.sqrt(c.hidden_size), tie_embeddings=True,
                     sandwich_norm=True, attn_softcap=c.attn_logit_softcapping or 0.0,
                     logit_softcap=c.final_logit_softcapping or 0.0, attn_scale=c.query_pre_attn_scalar ** -0.5,
                     sliding_window=c.sliding_window, layer_types=lt)


EXPORTS.update(define_family(
    "gemma2", dict(_GEMMA, hidden_size=2304, intermediate_size=9216, num_hidden_layers=26, num_attention_heads=8,
                   num_key_value_heads=4, query_pre_attn_scalar=256, sliding_window=4096, layer_types=None,
                   final_logit_softcapping=30.0, attn_logit_softcapping=50.0), _gemma2_spec,
    rules=[("post_attention_layernorm", "post_attn_out_layernorm")]))


def _gemma3_spec(c):
    n = c.num_hidden_layers
    pat = getattr(c, "sliding_window_pattern", 6) or 6
    lt = _layer_types(c, n) or tuple("full" if (i + 1) % pat == 0 else "sliding" for i in range(n))
    hd = c.head_dim
    glob = rope_args(c, hd)
    local = dict(glob, base=getattr(c, "rope_local_base_freq", 10000.0), rope_scaling=None)
    return base_spec(c, norm_offset=1.0, act=_gemma_act(c), embed_scale=math.sqrt(c.hidden_size), tie_embeddings=True,
                     sandwich_norm=True, qk_norm="rms_head", attn_scale=c.query_pre_attn_scalar ** -0.5,
                     sliding_window=c.sliding_window, layer_types=lt, rope=glob, rope_local=local,
                     attn_softcap=getattr(c, "attn_logit_softcapping", None) or 0.0,
                     logit_softcap=getattr(c, "final_logit_softcapping", None) or 0.0)


EXPORTS.update(define_family(
    "gemma3_text", dict(_GEMMA, vocab_size=262208, hidden_size=2304, intermediate_size=9216, num_hidden_layers=26,
                        num_attention_heads=8, num_key_value_heads=4, query_pre_attn_scalar=256, sliding_window=4096,
                        layer_types=None, rope_theta=1000000.0, rope_local_base_freq=10000.0,
                        sliding_window_pattern=6, max_position_embeddings=131072, final_logit_softcapping=None,
                        attn_logit_softcapping=None), _gemma3_spec, class_prefix="Gemma3Text",
    rules=[("post_attention_layernorm", "post_attn_out_layernorm")]))

# ---- phi3 (easydel/modules/phi3): checkpoints already hold fused qkv / gate_up -----------------
EXPORTS.update(define_family(
    "phi3", _d(vocab_size=32064, hidden_size=3072, intermediate_size=8192, rms_norm_eps=1e-5, sliding_window=None,
               original_max_position_embeddings=4096, partial_rotary_factor=1.0, pad_token_id=32000),
    lambda c: base_spec(c, sliding_window=getattr(c, "sliding_window", None),
                        rope=rope_args(c, c.hidden_size // c.num_attention_heads,
                                       partial=getattr(c, "partial_rotary_factor", 1.0))),
    hf_keeps_fused=("qkv_proj", "gate_up_proj")))

# ---- olmo / olmo2 / olmo3 (easydel/modules/olmo*) ----------------------------------------------
EXPORTS.update(define_family(
    "olmo", _d(vocab_size=50304, clip_qkv=None, max_position_embeddings=2048),
    lambda c: base_spec(c, norm="layer_noparam", clip_qkv=c.clip_qkv)))
EXPORTS.update(define_family(
    "olmo2", _d(vocab_size=50304, rms_norm_eps=1e-5, max_position_embeddings=2048),
    lambda c: base_spec(c, residual="post", qk_norm="rms_full")))


def _olmo3_spec(c):
    n = c.num_hidden_layers
    lt = _layer_types(c, n) or tuple("sliding" if (i + 1) % 4 else "full" for i in range(n))
    return base_spec(c, residual="post", qk_norm="rms_full", sliding_window=getattr(c, "sliding_window", None),
                     layer_types=lt)


EXPORTS.update(define_family("olmo3", _d(vocab_size=50304, rms_norm_eps=1e-5, sliding_window=4096, layer_types=None),
                             _olmo3_spec))

# ---- cohere (easydel/modules/cohere): parallel block, LayerNorm without bias, interleaved RoPE ---
EXPORTS.update(define_family(
    "cohere", _d(vocab_size=256000, hidden_size=8192, intermediate_size=22528, num_hidden_layers=40,
                 num_attention_heads=64, logit_scale=0.0625, layer_norm_eps=1e-5, use_qk_norm=False,
                 max_position_embeddings=8192, tie_word_embeddings=True),
    lambda c: base_spec(c, norm="layer", norm_bias=False, norm_eps=c.layer_norm_eps, residual="parallel",
                        shared_parallel_norm=True, logit_scale=c.logit_scale, tie_embeddings=True,
                        qk_norm="layer_perhead" if c.use_qk_norm else None,
                        rope=rope_args(c, c.hidden_size // c.num_attention_heads, neox=False)),
    layernorm_names=["input_layernorm", "norm"]))

# ---- stablelm (easydel/modules/stablelm): LayerNorm, partial rotary -------------------------------
EXPORTS.update(define_family(
    "stablelm", _d(vocab_size=50304, hidden_size=2560, intermediate_size=6912, layer_norm_eps=1e-5,
                   partial_rotary_factor=0.25, use_qkv_bias=False, qk_layernorm=False, use_parallel_residual=False),
    lambda c: base_spec(c, norm="layer", norm_eps=c.layer_norm_eps, attn_bias=c.use_qkv_bias, o_bias=False,
                        rope=rope_args(c, c.hidden_size // c.num_attention_heads, partial=c.partial_rotary_factor)),
    layernorm_names=["input_layernorm", "post_attention_layernorm", "norm"]))

# ---- starcoder2: LayerNorm + bias, plain GELU MLP ---------------------------------------------------
EXPORTS.update(define_family(
    "starcoder2", _d(vocab_size=49152, hidden_size=3072, intermediate_size=12288, num_hidden_layers=30,
                     num_attention_heads=24, num_key_value_heads=2, hidden_act="gelu_pytorch_tanh", norm_epsilon=1e-5,
                     use_bias=True, sliding_window=None, tie_word_embeddings=True),
    lambda c: base_spec(c, norm="layer", norm_eps=c.norm_epsilon, mlp="plain", mlp_bias=c.use_bias,
                        attn_bias=c.use_bias, o_bias=c.use_bias, sliding_window=c.sliding_window),
    rules=[("mlp.c_fc", "mlp.fc1"), ("mlp.c_proj", "mlp.fc2")],
    layernorm_names=["input_layernorm", "post_attention_layernorm", "norm"]))

# ---- glm / glm4 (easydel/modules/glm, glm4): half rotary, interleaved; fused gate_up in checkpoints --
_GLM = _d(vocab_size=151552, hidden_size=4096, intermediate_size=13696, num_hidden_layers=40, num_attention_heads=32,
          num_key_value_heads=2, head_dim=128, partial_rotary_factor=0.5, rms_norm_eps=1.5625e-07,
          attention_bias=True, max_position_embeddings=131072)
EXPORTS.update(define_family(
    "glm", _GLM, lambda c: base_spec(c, attn_bias=c.attention_bias, o_bias=False,
                                     rope=rope_args(c, c.head_dim, partial=c.partial_rotary_factor, neox=False)),
    hf_keeps_fused=("gate_up_proj",)))
EXPORTS.update(define_family(
    "glm4", _GLM, lambda c: base_spec(c, attn_bias=c.attention_bias, o_bias=False, sandwich_norm=True,
                                      rope=rope_args(c, c.head_dim, partial=c.partial_rotary_factor, neox=False)),
    hf_keeps_fused=("gate_up_proj",),
    rules=[("post_self_attn_layernorm", "post_attn_out_layernorm"),
           ("post_attention_layernorm", "pre_feedforward_layernorm"),
           ("post_mlp_layernorm", "post_feedforward_layernorm")]))


# ---- MoE families --------------------------------------------------------------------------------
def _mixtral_spec(c):
    return base_spec(c, sliding_window=getattr(c, "sliding_window", None),
                     moe=moe_spec(c, num_experts=c.num_local_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.intermediate_size, norm_topk=True,
                                  aux_coef=getattr(c, "router_aux_loss_coef", 0.0)))


EXPORTS.update(define_family(
    "mixtral", _d(intermediate_size=14336, num_key_value_heads=8, num_local_experts=8, num_experts_per_tok=2,
                  sliding_window=None, router_aux_loss_coef=0.001, output_router_logits=False,
                  max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=1e6),
    _mixtral_spec,
    rules=[("block_sparse_moe", "mlp"), (".w1.", ".gate_proj."), (".w3.", ".up_proj."), (".w2.", ".down_proj.")]))


def _qwen_moe_layers(c):
    n = c.num_hidden_layers
    only = set(getattr(c, "mlp_only_layers", None) or [])
    step = getattr(c, "decoder_sparse_step", 1) or 1
    return tuple(i for i in range(n) if i not in only and (i + 1) % step == 0)


def _qwen3_moe_spec(c):
    return base_spec(c, qk_norm="rms_head",
                     moe=moe_spec(c, num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob,
                                  layers=_qwen_moe_layers(c), aux_coef=c.router_aux_loss_coef))


EXPORTS.update(define_family(
    "qwen3_moe", _d(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=24,
                    num_attention_heads=32, num_key_value_heads=4, head_dim=128, max_position_embeddings=32768,
                    decoder_sparse_step=1, moe_intermediate_size=768, num_experts_per_tok=8, num_experts=128,
                    norm_topk_prob=False, output_router_logits=False, router_aux_loss_coef=0.001,
                    mlp_only_layers=None, use_sliding_window=False, sliding_window=None),
    _qwen3_moe_spec, class_prefix="Qwen3Moe"))


def _qwen2_moe_spec(c):
    return base_spec(c, attn_bias=True, o_bias=False,
                     moe=moe_spec(c, num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob,
                                  shared=c.shared_expert_intermediate_size, shared_gate=True,
                                  layers=_qwen_moe_layers(c), aux_coef=c.router_aux_loss_coef))


EXPORTS.update(define_family(
    "qwen2_moe", _d(vocab_size=151936, hidden_size=2048, intermediate_size=5632, num_hidden_layers=24,
                    num_attention_heads=16, num_key_value_heads=16, max_position_embeddings=32768,
                    decoder_sparse_step=1, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
                    num_experts_per_tok=4, num_experts=60, norm_topk_prob=False, output_router_logits=False,
                    router_aux_loss_coef=0.001, mlp_only_layers=None, use_sliding_window=False, sliding_window=4096),
    _qwen2_moe_spec, class_prefix="Qwen2Moe",
    rules=[("mlp.shared_expert.", "mlp.shared_experts.")]))

globals().update(EXPORTS)
__all__ = sorted(EXPORTS)


# ---- cohere2 (easydel/modules/cohere2): sliding layers rotate, every fourth (global) layer has no positions ----
def _cohere2_spec(c):
    n = c.num_hidden_layers
    pat = getattr(c, "sliding_window_pattern", 4) or 4
    lt = getattr(c, "layer_types", None)
    if lt:
        types = tuple("sliding" if "sliding" in t else "nope" for t in lt)
    else:
        types = tuple("nope" if (i + 1) % pat == 0 else "sliding" for i in range(n))
    return base_spec(c, norm="layer", norm_bias=False, norm_eps=c.layer_norm_eps, residual="parallel",
                     shared_parallel_norm=True, logit_scale=c.logit_scale, tie_embeddings=True,
                     sliding_window=c.sliding_window, layer_types=types,
                     rope=rope_args(c, c.hidden_size // c.num_attention_heads, neox=False))


EXPORTS.update(define_family(
    "cohere2", _d(vocab_size=256000, hidden_size=8192, intermediate_size=22528, num_hidden_layers=40,
                  num_attention_heads=64, logit_scale=0.0625, layer_norm_eps=1e-5, sliding_window=4096,
                  sliding_window_pattern=4, layer_types=None, max_position_embeddings=8192, tie_word_embeddings=True),
    _cohere2_spec, layernorm_names=["input_layernorm", "norm"]))


# ---- deepseek_v2 / deepseek_v3 (easydel/modules/deepseek_v2, deepseek_v3): latent attention + routed experts ------
def _yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def _mla_args(c) -> dict:
    qk = c.qk_nope_head_dim + c.qk_rope_head_dim
    scale = qk ** -0.5
    rs = getattr(c, "rope_scaling", None)
    if isinstance(rs, dict) and rs.get("mscale_all_dim"):
        scale = scale * _yarn_mscale(rs.get("factor", 1.0), rs["mscale_all_dim"]) ** 2
    return dict(q_lora_rank=c.q_lora_rank, kv_lora_rank=c.kv_lora_rank, qk_nope_head_dim=c.qk_nope_head_dim,
                qk_rope_head_dim=c.qk_rope_head_dim, v_head_dim=c.v_head_dim, scale=scale,
                rope_interleave=getattr(c, "rope_interleave", True))


def _dense_then_moe(c, freq_attr="moe_layer_freq"):
    n = c.num_hidden_layers
    kinds = getattr(c, "mlp_layer_types", None)
    if kinds:       # explicit per-layer list ("dense" / "sparse")
        return tuple(i for i, k in enumerate(kinds) if k == "sparse")
    freq = getattr(c, freq_attr, 1) or 1
    return tuple(i for i in range(n) if i >= c.first_k_dense_replace and i % freq == 0)


def _deepseek_v3_spec(c):
    return base_spec(
        c, head_dim=c.qk_rope_head_dim, rope=rope_args(c, c.qk_rope_head_dim), mla=_mla_args(c),
        moe=moe_spec(c, num_experts=c.n_routed_experts, top_k=c.num_experts_per_tok,
                     intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob,
                     shared=c.moe_intermediate_size * (c.n_shared_experts or 0), layers=_dense_then_moe(c),
                     scoring="sigmoid", routed_scaling_factor=c.routed_scaling_factor, n_group=c.n_group,
                     topk_group=c.topk_group, use_score_bias=True))


_DSV3 = _d(vocab_size=129280, hidden_size=7168, intermediate_size=18432, moe_intermediate_size=2048,
           num_hidden_layers=61, num_attention_heads=128, num_key_value_heads=128, n_shared_experts=1,
           n_routed_experts=256, routed_scaling_factor=2.5, kv_lora_rank=512, q_lora_rank=1536, qk_rope_head_dim=64,
           v_head_dim=128, qk_nope_head_dim=128, n_group=8, topk_group=4, num_experts_per_tok=8,
           first_k_dense_replace=3, norm_topk_prob=True, rope_interleave=True, moe_layer_freq=1,
           max_position_embeddings=4096)
_DSV3.pop("head_dim", None)
EXPORTS.update(define_family(
    "deepseek_v3", _DSV3, _deepseek_v3_spec, class_prefix="DeepseekV3",
    rules=[("mlp.gate.e_score_correction_bias", "mlp.e_score_correction_bias")], with_classifier=False))


def _deepseek_v2_spec(c):
    grouped = getattr(c, "topk_method", "greedy") == "group_limited_greedy"
    return base_spec(
        c, head_dim=c.qk_rope_head_dim, rope=rope_args(c, c.qk_rope_head_dim), mla=_mla_args(c),
        moe=moe_spec(c, num_experts=c.n_routed_experts, top_k=c.num_experts_per_tok,
                     intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob,
                     shared=c.moe_intermediate_size * (c.n_shared_experts or 0), layers=_dense_then_moe(c),
                     scoring="softmax", routed_scaling_factor=c.routed_scaling_factor,
                     n_group=c.n_group if grouped else 1, topk_group=c.topk_group if grouped else 1))


_DSV2 = dict(_DSV3, vocab_size=102400, hidden_size=4096, intermediate_size=11008, moe_intermediate_size=1407,
             num_hidden_layers=30, num_attention_heads=32, num_key_value_heads=32, n_shared_experts=2,
             n_routed_experts=64, routed_scaling_factor=1.0, topk_method="greedy", n_group=1, topk_group=1,
             num_experts_per_tok=6, first_k_dense_replace=1, norm_topk_prob=False, max_position_embeddings=2048)
EXPORTS.update(define_family("deepseek_v2", _DSV2, _deepseek_v2_spec, class_prefix="DeepseekV2",
                             with_classifier=False))


# ---- glm4_moe (easydel/modules/glm4_moe): GQA with partial rotary + DeepSeek-style routed experts -------------------
def _glm4_moe_spec(c):
    return base_spec(
        c, attn_bias=c.attention_bias, o_bias=False, qk_norm="rms_head" if c.use_qk_norm else None,
        rope=rope_args(c, c.head_dim, partial=c.partial_rotary_factor),
        moe=moe_spec(c, num_experts=c.n_routed_experts, top_k=c.num_experts_per_tok,
                     intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob,
                     shared=c.moe_intermediate_size * (c.n_shared_experts or 0),
                     layers=tuple(range(c.first_k_dense_replace, c.num_hidden_layers)), scoring="sigmoid",
                     routed_scaling_factor=c.routed_scaling_factor, n_group=c.n_group, topk_group=c.topk_group,
                     use_score_bias=True))


EXPORTS.update(define_family(
    "glm4_moe", _d(vocab_size=151552, hidden_size=4096, intermediate_size=10944, num_hidden_layers=46,
                   num_attention_heads=96, num_key_value_heads=8, head_dim=128, partial_rotary_factor=0.5,
                   rms_norm_eps=1e-5, attention_bias=False, moe_intermediate_size=1408, num_experts_per_tok=8,
                   n_shared_experts=1, n_routed_experts=128, routed_scaling_factor=1.0, n_group=1, topk_group=1,
                   first_k_dense_replace=1, norm_topk_prob=True, use_qk_norm=False, max_position_embeddings=131072),
    _glm4_moe_spec, class_prefix="Glm4Moe",
    rules=[("mlp.gate.e_score_correction_bias", "mlp.e_score_correction_bias")], with_classifier=False))



# ---- exaone4 (easydel/modules/exaone4): post-norm blocks, per-head QK norm, local layers rotate / global layers do not
def _exaone4_spec(c):
    n = c.num_hidden_layers
    if c.sliding_window:
        lt = getattr(c, "layer_types", None)
        pat = getattr(c, "sliding_window_pattern", 4) or 4
        types = tuple(("sliding" if "sliding" in t else "nope") for t in lt) if lt else \
            tuple("nope" if (i + 1) % pat == 0 else "sliding" for i in range(n))
    else:
        types = None
    return base_spec(c, residual="post", qk_norm="rms_head", sliding_window=c.sliding_window, layer_types=types)


EXPORTS.update(define_family(
    "exaone4", _d(vocab_size=102400, hidden_size=4096, intermediate_size=16384, rms_norm_eps=1e-5,
                  sliding_window=4096, sliding_window_pattern=4, layer_types=None, max_position_embeddings=2048),
    _exaone4_spec))



# ---- gpt_oss (easydel/modules/gpt_oss): attention sinks, alternating sliding / full layers, YaRN; top-k router with
# ---- bias; experts with biases and the clamped x*sigmoid(1.702x) gate. Hugging Face stores the expert tensors as
# ---- [E, in, 2F] with gate / up columns interleaved; here they are [E, 2F, in] with the gate rows first.
def _gpt_oss_spec(c):
    n = c.num_hidden_layers
    lt = _layer_types(c, n) or tuple("sliding" if i % 2 == 0 else "full" for i in range(n))
    return base_spec(c, use_sinks=True, attn_bias=True, o_bias=True, sliding_window=c.sliding_window, layer_types=lt,
                     moe=moe_spec(c, num_experts=c.num_local_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.intermediate_size, norm_topk=True, router_bias=True,
                                  expert_bias=True, expert_act="gptoss_swiglu",
                                  aux_coef=getattr(c, "router_aux_loss_coef", 0.0)))


def _gpt_oss_in(model, sd):
    out = {}
    for k, t in sd.items():
        if k.endswith("mlp.experts.gate_up_proj"):
            w = t.transpose(1, 2)                                    # [E, 2F, in], rows interleaved
            out[k[:-len("experts.gate_up_proj")] + "gate_up_proj.weight"] = torch.cat([w[:, 0::2], w[:, 1::2]], 1)
        elif k.endswith("mlp.experts.gate_up_proj_bias"):
            out[k[:-len("experts.gate_up_proj_bias")] + "gate_up_proj.bias"] = torch.cat([t[:, 0::2], t[:, 1::2]], 1)
        elif k.endswith("mlp.experts.down_proj"):
            out[k[:-len("experts.down_proj")] + "down_proj.weight"] = t.transpose(1, 2)
        elif k.endswith("mlp.experts.down_proj_bias"):
            out[k[:-len("experts.down_proj_bias")] + "down_proj.bias"] = t
        else:
            out[k] = t
    return out


def _interleave(gate, up, dim):
    return torch.stack([gate, up], dim + 1).flatten(dim, dim + 1)


def _gpt_oss_out(model, sd):
    out = {}
    for k, t in sd.items():
        if k.endswith("mlp.gate_up_proj.weight"):
            f = t.shape[1] // 2
            out[k[:-len("gate_up_proj.weight")] + "experts.gate_up_proj"] = \
                _interleave(t[:, :f], t[:, f:], 1).transpose(1, 2).contiguous()
        elif k.endswith("mlp.gate_up_proj.bias"):
            f = t.shape[1] // 2
            out[k[:-len("gate_up_proj.bias")] + "experts.gate_up_proj_bias"] = _interleave(t[:, :f], t[:, f:], 1)
        elif k.endswith("mlp.down_proj.weight") and t.dim() == 3:
            out[k[:-len("down_proj.weight")] + "experts.down_proj"] = t.transpose(1, 2).contiguous()
        elif k.endswith("mlp.down_proj.bias") and t.dim() == 2:
            out[k[:-len("down_proj.bias")] + "experts.down_proj_bias"] = t
        else:
            out[k] = t
    return out


EXPORTS.update(define_family(
    "gpt_oss", _d(vocab_size=201088, hidden_size=2880, intermediate_size=2880, num_hidden_layers=36,
                  num_attention_heads=64, num_key_value_heads=8, head_dim=64, num_local_experts=128,
                  num_experts_per_tok=4, sliding_window=128, rms_norm_eps=1e-5, attention_bias=True,
                  rope_theta=150000.0, max_position_embeddings=131072, initial_context_length=4096, layer_types=None,
                  router_aux_loss_coef=0.9, output_router_logits=False,
                  rope_scaling={"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                "truncate": False, "original_max_position_embeddings": 4096}),
    _gpt_oss_spec, class_prefix="GptOss", rules=[("mlp.router.", "mlp.gate.")], tensor_in=_gpt_oss_in,
    tensor_out=_gpt_oss_out, hf_keeps_fused=("experts",)))



# ---- qwen3_next (easydel/modules/qwen3_next): three Gated-DeltaNet layers per gated full-attention layer, (1 + w)
# ---- RMSNorm, rotary on a quarter of the head, MoE with a gated shared expert ----
def _qwen3_next_spec(c):
    n = c.num_hidden_layers
    lt = getattr(c, "layer_types", None)
    interval = getattr(c, "full_attention_interval", 4) or 4
    types = tuple("linear" if "linear" in t else "full" for t in lt) if lt else \
        tuple("full" if (i + 1) % interval == 0 else "linear" for i in range(n))
    hd = c.head_dim
    params = getattr(c, "rope_parameters", None) or {}
    partial = getattr(c, "partial_rotary_factor", None) or params.get("partial_rotary_factor", 0.25)
    moe = None
    if c.num_experts > 0:
        moe = moe_spec(c, num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                       intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob,
                       shared=c.shared_expert_intermediate_size, shared_gate=True, layers=_qwen_moe_layers(c),
                       aux_coef=c.router_aux_loss_coef)
    return base_spec(c, qk_norm="rms_head", norm_offset=1.0, layer_types=types, attn_output_gate=True,
                     rope=rope_args(c, hd, partial=partial),
                     linear_attn=dict(num_k_heads=c.linear_num_key_heads, num_v_heads=c.linear_num_value_heads,
                                      head_k_dim=c.linear_key_head_dim, head_v_dim=c.linear_value_head_dim,
                                      conv_kernel=c.linear_conv_kernel_dim), moe=moe)


EXPORTS.update(define_family(
    "qwen3_next", _d(vocab_size=151936, hidden_size=2048, intermediate_size=5632, num_hidden_layers=48,
                     num_attention_heads=16, num_key_value_heads=2, head_dim=256, partial_rotary_factor=0.25,
                     max_position_embeddings=32768, rope_theta=10000000.0, linear_conv_kernel_dim=4,
                     linear_key_head_dim=128, linear_value_head_dim=128, linear_num_key_heads=16,
                     linear_num_value_heads=32, decoder_sparse_step=1, moe_intermediate_size=512,
                     shared_expert_intermediate_size=512, num_experts_per_tok=10, num_experts=512,
                     norm_topk_prob=True, output_router_logits=False, router_aux_loss_coef=0.001,
                     mlp_only_layers=None, layer_types=None, full_attention_interval=4),
    _qwen3_next_spec, class_prefix="Qwen3Next", rules=[("mlp.shared_expert.", "mlp.shared_experts.")]))



# ---- llama4 text (easydel/modules/llama4): rotary layers attend inside 8192-token blocks and L2-normalise q / k,
# ---- every fourth layer has no positions and a length-dependent query temperature; top-1 sigmoid router whose score
# ---- scales the expert input; a shared expert beside the routed ones. Expert tensors are stored [E, in, out].
def _llama4_spec(c):
    n = c.num_hidden_layers
    nope = getattr(c, "no_rope_layers", None) or [int((i + 1) % 4 != 0) for i in range(n)]
    types = tuple("full" if r else "nope" for r in nope)
    step = getattr(c, "interleave_moe_layer_step", 1) or 1
    moe_layers = getattr(c, "moe_layers", None)
    if moe_layers is None:
        moe_layers = list(range(step - 1, n, step))
    return base_spec(c, intermediate_size=c.intermediate_size_mlp, layer_types=types,
                     rope=rope_args(c, c.head_dim, neox=False),
                     qk_norm="l2_post_rope" if c.use_qk_norm else None, qk_norm_rope_only=True,
                     attn_chunk_size=c.attention_chunk_size,
                     attn_temp_tuning=(c.attn_scale, c.floor_scale) if c.attn_temperature_tuning else None,
                     moe=moe_spec(c, num_experts=c.num_local_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.intermediate_size, norm_topk=False, scoring="sigmoid",
                                  shared=c.intermediate_size, layers=tuple(moe_layers), scale_input=True,
                                  aux_coef=getattr(c, "router_aux_loss_coef", 0.0)))


def _fused_experts_in(model, sd):
    """``...experts.gate_up_proj`` [E, in, 2F] / ``...experts.down_proj`` [E, F, out] -> stacked ``.weight`` [E, out, in]."""
    out = {}
    for k, t in sd.items():
        if k.endswith(".experts.gate_up_proj") or k.endswith(".experts.down_proj"):
            head, leaf = k.rsplit(".experts.", 1)
            out[f"{head}.{leaf}.weight"] = t.transpose(1, 2)
        else:
            out[k] = t
    return out


def _fused_experts_out(model, sd):
    out = {}
    for k, t in sd.items():
        if t.dim() == 3 and (k.endswith(".gate_up_proj.weight") or k.endswith(".down_proj.weight")):
            head, leaf, _ = k.rsplit(".", 2)
            out[f"{head}.experts.{leaf}"] = t.transpose(1, 2).contiguous()
        else:
            out[k] = t
    return out


EXPORTS.update(define_family(
    "llama4_text", _d(vocab_size=202048, hidden_size=5120, intermediate_size=8192, intermediate_size_mlp=16384,
                      num_hidden_layers=48, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                      rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=131072, num_experts_per_tok=1,
                      num_local_experts=16, moe_layers=None, interleave_moe_layer_step=1, use_qk_norm=True,
                      output_router_logits=False, router_aux_loss_coef=0.001, router_jitter_noise=0.0,
                      no_rope_layers=None, no_rope_layer_interval=4, attention_chunk_size=8192,
                      attn_temperature_tuning=True, floor_scale=8192, attn_scale=0.1, layer_types=None),
    _llama4_spec, class_prefix="Llama4Text",
    rules=[("feed_forward.router.", "mlp.gate."), ("feed_forward.shared_expert.", "mlp.shared_experts."),
           ("feed_forward.", "mlp.")],
    tensor_in=_fused_experts_in, tensor_out=_fused_experts_out, hf_keeps_fused=("experts",)))



# ---- phimoe (easydel/modules/phimoe): Mixtral block with LayerNorm (weights + biases) and sparsemixer routing ----
def _phimoe_spec(c):
    return base_spec(c, norm="layer", norm_bias=True, norm_eps=c.rms_norm_eps,
                     sliding_window=getattr(c, "sliding_window", None), lm_head_bias=getattr(c, "lm_head_bias", False),
                     moe=moe_spec(c, num_experts=c.num_local_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.intermediate_size, norm_topk=False, scoring="sparsemixer",
                                  router_jitter_eps=c.router_jitter_noise, aux_coef=c.router_aux_loss_coef))


EXPORTS.update(define_family(
    "phimoe", _d(vocab_size=32064, hidden_size=4096, intermediate_size=6400, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=131072, rms_norm_eps=1e-5,
                 rope_theta=1000000.0, sliding_window=None, num_experts_per_tok=2, num_local_experts=16,
                 output_router_logits=False, router_aux_loss_coef=0.001, router_jitter_noise=0.01,
                 input_jitter_noise=0.0, attention_bias=False, lm_head_bias=False),
    _phimoe_spec, class_prefix="Phimoe", rules=[("mlp.router.", "mlp.gate.")]))



# ---- glm4_moe_lite (easydel/modules/glm4_moe_lite): the DeepSeek-V3 block (latent attention, sigmoid-scored experts
# ---- with a score-correction bias, one shared expert) at GLM sizes ----
_GLM4_LITE = dict(_DSV3, vocab_size=154880, hidden_size=2048, intermediate_size=10240, moe_intermediate_size=1536,
                  num_hidden_layers=47, num_attention_heads=20, num_key_value_heads=20, n_shared_experts=1,
                  n_routed_experts=64, routed_scaling_factor=1.8, kv_lora_rank=512, q_lora_rank=768,
                  qk_rope_head_dim=64, v_head_dim=256, qk_nope_head_dim=192, n_group=1, topk_group=1,
                  num_experts_per_tok=4, first_k_dense_replace=1, norm_topk_prob=True, rope_interleave=True,
                  max_position_embeddings=202752, rms_norm_eps=1e-5, mlp_layer_types=None)
EXPORTS.update(define_family(
    "glm4_moe_lite", _GLM4_LITE, _deepseek_v3_spec, class_prefix="Glm4MoeLite",
    rules=[("mlp.gate.e_score_correction_bias", "mlp.e_score_correction_bias")], with_classifier=False))



# ---- qwen3_5 text (easydel/modules/qwen3_5): the Qwen3-Next hybrid with a dense MLP and un-grouped DeltaNet
# ---- projections; text-only inputs give all three rotary streams the same position, i.e. plain partial rotary ----
def _qwen3_5_spec(c):
    spec = _qwen3_next_spec(c)
    spec.linear_attn = dict(spec.linear_attn, layout="flat")
    return spec


EXPORTS.update(define_family(
    "qwen3_5_text", _d(vocab_size=248320, hidden_size=4096, intermediate_size=12288, num_hidden_layers=32,
                       num_attention_heads=16, num_key_value_heads=4, head_dim=256, partial_rotary_factor=0.25,
                       max_position_embeddings=32768, rope_theta=10000000.0, linear_conv_kernel_dim=4,
                       linear_key_head_dim=128, linear_value_head_dim=128, linear_num_key_heads=16,
                       linear_num_value_heads=32, num_experts=0, layer_types=None, full_attention_interval=4),
    _qwen3_5_spec, class_prefix="Qwen3_5Text"))


EXPORTS.update(define_family(
    "qwen3_5_moe_text", _d(vocab_size=248320, hidden_size=2048, intermediate_size=5632, num_hidden_layers=40,
                           num_attention_heads=16, num_key_value_heads=2, head_dim=256, partial_rotary_factor=0.25,
                           max_position_embeddings=32768, rope_theta=10000000.0, linear_conv_kernel_dim=4,
                           linear_key_head_dim=128, linear_value_head_dim=128, linear_num_key_heads=16,
                           linear_num_value_heads=32, decoder_sparse_step=1, moe_intermediate_size=512,
                           shared_expert_intermediate_size=512, num_experts_per_tok=8, num_experts=256,
                           norm_topk_prob=True, output_router_logits=False, router_aux_loss_coef=0.001,
                           mlp_only_layers=None, layer_types=None, full_attention_interval=4),
    _qwen3_5_spec, class_prefix="Qwen3_5MoeText", rules=[("mlp.shared_expert.", "mlp.shared_experts.")]))



# ---- falcon_h1 (easydel/modules/falcon_h1): every block runs attention and a Mamba-2 mixer side by side on the same
# ---- normalised input and sums them; fixed muP multipliers sit on embeddings, keys, both branches, the MLP and logits
def _falcon_h1_spec(c):
    hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
    d_ssm = c.mamba_d_ssm if c.mamba_d_ssm is not None else int(c.mamba_expand * c.hidden_size)
    return base_spec(
        c, head_dim=hd, attn_scale=c.key_multiplier / math.sqrt(hd), embedding_multiplier=c.embedding_multiplier,
        logit_scale=c.lm_head_multiplier, mlp_bias=c.mlp_bias, attn_bias=c.attention_bias, o_bias=c.attention_bias,
        branch_multipliers=(c.attention_in_multiplier, c.attention_out_multiplier, c.ssm_out_multiplier),
        mlp_multipliers=tuple(c.mlp_multipliers),
        ssm_branch=dict(d_ssm=d_ssm, num_heads=c.mamba_n_heads, head_dim=c.mamba_d_head, n_groups=c.mamba_n_groups,
                        d_state=c.mamba_d_state, d_conv=c.mamba_d_conv, conv_bias=c.mamba_conv_bias,
                        proj_bias=c.mamba_proj_bias, rms_norm=c.mamba_rms_norm,
                        norm_before_gate=c.mamba_norm_before_gate, multipliers=tuple(c.ssm_multipliers),
                        in_multiplier=c.ssm_in_multiplier))


EXPORTS.update(define_family(
    "falcon_h1", _d(vocab_size=128000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                    num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=8192, rms_norm_eps=1e-5,
                    rope_theta=100000.0, mamba_d_ssm=1024, mamba_n_heads=128, mamba_d_head=64, mamba_n_groups=1,
                    mamba_d_state=256, mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=256, mamba_conv_bias=True,
                    mamba_proj_bias=False, mamba_norm_before_gate=True, mamba_rms_norm=False, projectors_bias=False,
                    lm_head_multiplier=1.0, embedding_multiplier=1.0, mlp_multipliers=[1.0, 1.0], key_multiplier=1.0,
                    attention_out_multiplier=1.0, attention_in_multiplier=1.0, ssm_multipliers=[1.0] * 5,
                    ssm_in_multiplier=1.0, ssm_out_multiplier=1.0, mlp_bias=False),
    _falcon_h1_spec, class_prefix="FalconH1",
    rules=[(".feed_forward.", ".mlp."), (".pre_ff_layernorm.", ".post_attention_layernorm."),
           ("model.final_layernorm.", "model.norm.")], with_classifier=False))



# ---- minimax (easydel/modules/minimax): lightning (decayed linear) attention layers interleaved with softmax layers,
# ---- experts in every layer, and residual branches that start from the *normalised* input with fixed alpha / beta ----
def _minimax_spec(c):
    n = c.num_hidden_layers
    lt = getattr(c, "layer_types", None)
    types = tuple("lightning" if "linear" in t else "full" for t in lt) if lt else \
        tuple("full" if (i + 1) % 2 == 0 else "lightning" for i in range(n))
    return base_spec(c, layer_types=types, lightning=dict(block_size=c.block_size),
                     normed_residual=dict(attn=(c.full_attn_alpha_factor, c.full_attn_beta_factor),
                                          lightning=(c.linear_attn_alpha_factor, c.linear_attn_beta_factor),
                                          mlp=(c.mlp_alpha_factor, c.mlp_beta_factor)),
                     moe=moe_spec(c, num_experts=c.num_local_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.intermediate_size, norm_topk=True,
                                  aux_coef=c.router_aux_loss_coef))


EXPORTS.update(define_family(
    "minimax", _d(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                  num_attention_heads=32, num_key_value_heads=8, head_dim=None, max_position_embeddings=4096 * 32,
                  rms_norm_eps=1e-5, rope_theta=1e6, sliding_window=None, num_experts_per_tok=2, num_local_experts=8,
                  output_router_logits=False, router_aux_loss_coef=0.001, router_jitter_noise=0.0, layer_types=None,
                  block_size=256, full_attn_alpha_factor=1, full_attn_beta_factor=1, linear_attn_alpha_factor=1,
                  linear_attn_beta_factor=1, mlp_alpha_factor=1, mlp_beta_factor=1),
    _minimax_spec, class_prefix="MiniMax", rules=[(".self_attn.qkv_proj.", ".self_attn.lqkv.")],
    with_classifier=False))



# ---- kimi_linear (easydel/modules/kimi_linear): Kimi delta attention layers (1-indexed ``kda_layers``) between latent
# ---- (MLA) attention layers without positions, DeepSeek-V3 style sigmoid-routed experts with shared experts ----
def _kimi_linear_spec(c):
    n = c.num_hidden_layers
    la = c.linear_attn_config or {}
    kda = set(la.get("kda_layers") or [])
    types = tuple("kda" if (i + 1) in kda else "full" for i in range(n))
    moe = None
    if c.num_experts:
        layers = tuple(i for i in range(n) if i >= c.first_k_dense_replace and i % (c.moe_layer_freq or 1) == 0)
        grouped = bool(c.use_grouped_topk)
        moe = moe_spec(c, num_experts=c.num_experts, top_k=c.num_experts_per_token,
                       intermediate=c.moe_intermediate_size, norm_topk=c.moe_renormalize,
                       shared=c.moe_intermediate_size * (c.num_shared_experts or 0), layers=layers,
                       scoring="sigmoid" if c.moe_router_activation_func == "sigmoid" else "softmax",
                       routed_scaling_factor=c.routed_scaling_factor, n_group=c.num_expert_group if grouped else 1,
                       topk_group=c.topk_group if grouped else 1, use_score_bias=True)
    mla = dict(_mla_args(c), use_rope=not c.mla_use_nope)
    return base_spec(c, head_dim=c.qk_rope_head_dim, rope=rope_args(c, c.qk_rope_head_dim), mla=mla, moe=moe,
                     layer_types=types,
                     linear_attn=dict(num_heads=la.get("num_heads", c.num_attention_heads),
                                      head_k_dim=la.get("head_k_dim", la.get("head_dim", 128)),
                                      head_v_dim=la.get("head_v_dim", la.get("head_dim", 128)),
                                      d_conv=la.get("short_conv_kernel_size", la.get("d_conv", 4)),
                                      gate_low_rank_dim=la.get("gate_low_rank_dim", 128)))


_KIMI = _d(vocab_size=163840, hidden_size=2304, intermediate_size=9216, num_hidden_layers=27, num_attention_heads=32,
           num_key_value_heads=32, rms_norm_eps=1e-5, q_lora_rank=None, kv_lora_rank=512, qk_nope_head_dim=128,
           qk_rope_head_dim=64, v_head_dim=128, mla_use_nope=True, num_experts=256, num_experts_per_token=8,
           moe_renormalize=True, num_shared_experts=1, routed_scaling_factor=2.446, moe_router_activation_func="sigmoid",
           moe_intermediate_size=1024, first_k_dense_replace=1, moe_layer_freq=1, use_grouped_topk=True,
           num_expert_group=1, topk_group=1, num_nextn_predict_layers=0, max_position_embeddings=1048576,
           linear_attn_config=None, rope_interleave=True)
_KIMI.pop("head_dim", None)
_KIMI_W = {"w1": "gate_proj", "w3": "up_proj", "w2": "down_proj"}
_KIMI_P = {v: k for k, v in _KIMI_W.items()}
_KIMI_IN = re.compile(r"\.experts\.(\d+)\.(w[123])\.")
_KIMI_DENSE = re.compile(r"\.block_sparse_moe\.(gate_proj|up_proj|down_proj)\.")   # dense layers keep ``mlp``
_KIMI_OUT = re.compile(r"\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.")
EXPORTS.update(define_family(
    "kimi_linear", _KIMI, _kimi_linear_spec, class_prefix="KimiLinear",
    rules=[(".block_sparse_moe.gate.e_score_correction_bias", ".mlp.e_score_correction_bias"),
           (".block_sparse_moe", ".mlp")],
    # routed experts are stored as experts.N.w1 / w3 / w2 (gate / up / down); shared and dense MLPs use the long names
    tensor_in=lambda model, sd: {_KIMI_IN.sub(lambda m: f".experts.{m.group(1)}.{_KIMI_W[m.group(2)]}.", k): v
                                 for k, v in sd.items()},
    tensor_out=lambda model, sd: {_KIMI_DENSE.sub(r".mlp.\1.", _KIMI_OUT.sub(
        lambda m: f".experts.{m.group(1)}.{_KIMI_P[m.group(2)]}.", k)): v for k, v in sd.items()},
    with_classifier=False))



# ---- glm4v_text (the language half of easydel/modules/glm4v, glm46v): the GLM-4 block with QKV biases always on and
# ---- the rotary fraction / three-stream sections carried in the rope parameters ----
def _glm4v_text_spec(c):
    rp = getattr(c, "rope_parameters", None) or getattr(c, "rope_scaling", None) or {}
    partial = getattr(c, "partial_rotary_factor", None) or rp.get("partial_rotary_factor", 1.0)
    hd = c.hidden_size // c.num_attention_heads
    return base_spec(c, head_dim=hd, attn_bias=True, o_bias=False, sandwich_norm=True,
                     rope=rope_args(c, hd, partial=partial, neox=False))


EXPORTS.update(define_family(
    "glm4v_text", _d(vocab_size=151552, hidden_size=4096, intermediate_size=13696, num_hidden_layers=40,
                     num_attention_heads=32, num_key_value_heads=2, rms_norm_eps=1e-5, max_position_embeddings=32768,
                     partial_rotary_factor=None),
    _glm4v_text_spec, class_prefix="Glm4vText", hf_keeps_fused=("gate_up_proj",),
    rules=[("post_self_attn_layernorm", "post_attn_out_layernorm"),
           ("post_attention_layernorm", "pre_feedforward_layernorm"),
           ("post_mlp_layernorm", "post_feedforward_layernorm")], with_classifier=False))



# ---- glm_moe_dsa (easydel/modules/glm_moe_dsa): the GLM-4-MoE-Lite block whose latent attention only looks at the
# ---- ``index_topk`` keys a small scorer (own projections, ReLU-weighted multi-head dot products) ranks highest ----
def _glm_moe_dsa_spec(c):
    spec = _deepseek_v3_spec(c)
    # rotary pairs are stored half-split in these checkpoints (no de-interleaving as in DeepSeek-V3)
    spec.mla = dict(spec.mla, rope_interleave=False,
                    indexer=dict(n_heads=c.index_n_heads, head_dim=c.index_head_dim, topk=c.index_topk))
    return spec


EXPORTS.update(define_family(
    "glm_moe_dsa", dict(_GLM4_LITE, vocab_size=154880, hidden_size=6144, intermediate_size=12288,
                        moe_intermediate_size=2048, num_hidden_layers=78, num_attention_heads=64,
                        num_key_value_heads=64, n_routed_experts=256, routed_scaling_factor=2.5, kv_lora_rank=512,
                        q_lora_rank=2048, qk_rope_head_dim=64, v_head_dim=256, qk_nope_head_dim=192,
                        num_experts_per_tok=8, first_k_dense_replace=3, index_topk=2048, index_head_dim=128,
                        index_n_heads=32),
    _glm_moe_dsa_spec, class_prefix="GlmMoeDsa",
    rules=[("mlp.gate.e_score_correction_bias", "mlp.e_score_correction_bias")], with_classifier=False))

globals().update(EXPORTS)
__all__ = sorted(EXPORTS)
