"""GPT-2 era decoder families: learned positions, LayerNorm, parallel residuals, fused QKV layouts.

Covers easydel/modules/{gpt2,gpt_neox,gpt_j,opt,phi,falcon}. Their checkpoints differ from the
Llama layout mostly in naming and in how the fused query/key/value matrix is ordered, so each block
below is an ArchSpec plus a pair of tensor hooks that reorder or transpose those matrices.
"""

from __future__ import annotations

import torch

from ._base.decoder import ArchSpec
from ._base.families import define_family, rope_args

EXPORTS: dict[str, type] = {}
_LN = ["input_layernorm", "post_attention_layernorm", "norm"]


def _map_tensors(sd: dict, suffixes: tuple[str, ...], fn) -> dict:
    return {k: (fn(k, v) if k.endswith(suffixes) else v) for k, v in sd.items()}


# ---- gpt2 (easydel/modules/gpt2): Conv1D weights are stored (in, out) ---------------------------
_GPT2_CONV = ("attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight")
_GPT2_RULES = [("transformer.wte.", "model.embed_tokens."), ("transformer.wpe.", "model.embed_positions."),
               ("transformer.ln_f.", "model.norm."), ("transformer.h.", "model.layers."),
               (".ln_1.", ".input_layernorm."), (".ln_2.", ".post_attention_layernorm."),
               (".attn.c_attn.", ".self_attn.qkv_proj."), (".attn.c_proj.", ".self_attn.o_proj."),
               (".mlp.c_fc.", ".mlp.fc1."), (".mlp.c_proj.", ".mlp.fc2.")]


def _gpt2_spec(c) -> ArchSpec:
    inner = c.n_inner if getattr(c, "n_inner", None) else 4 * c.n_embd
    return ArchSpec(hidden_size=c.n_embd, num_layers=c.n_layer, num_heads=c.n_head, num_kv_heads=c.n_head,
                    head_dim=c.n_embd // c.n_head, intermediate_size=inner, vocab_size=c.vocab_size,
                    max_position=c.n_positions, norm="layer", norm_eps=c.layer_norm_epsilon,
                    act=c.activation_function, mlp="plain", mlp_bias=True, attn_bias=True, o_bias=True, rope=None,
                    pos_emb="learned", tie_embeddings=True, init_std=c.initializer_range)


def _transpose(_, v):
    return v.t().contiguous()


EXPORTS.update(define_family(
    "gpt2", dict(vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12, n_inner=None,
                 activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                 layer_norm_epsilon=1e-5, initializer_range=0.02, scale_attn_weights=True, use_cache=True,
                 bos_token_id=50256, eos_token_id=50256, tie_word_embeddings=True),
    _gpt2_spec, class_prefix="GPT2", rules=_GPT2_RULES,
    tensor_in=lambda m, sd: _map_tensors(sd, _GPT2_CONV, _transpose),
    tensor_out=lambda m, sd: _map_tensors(sd, _GPT2_CONV, _transpose),
    hf_keeps_fused=("qkv_proj",), layernorm_names=_LN,
    attribute_map={"hidden_size": "n_embd", "max_position_embeddings": "n_positions",
                   "num_attention_heads": "n_head", "num_hidden_layers": "n_layer"}))


# ---- gpt_neox (easydel/modules/gpt_neox): QKV rows ordered [head][q|k|v][head_dim] ---------------
def _neox_spec(c) -> ArchSpec:
    hd = c.hidden_size // c.num_attention_heads
    return ArchSpec(hidden_size=c.hidden_size, num_layers=c.num_hidden_layers, num_heads=c.num_attention_heads,
                    num_kv_heads=c.num_attention_heads, head_dim=hd, intermediate_size=c.intermediate_size,
                    vocab_size=c.vocab_size, max_position=c.max_position_embeddings, norm="layer",
                    norm_eps=c.layer_norm_eps, act=c.hidden_act, mlp="plain", mlp_bias=True,
                    attn_bias=c.attention_bias, o_bias=c.attention_bias,
                    rope=rope_args(c, hd, partial=c.rotary_pct, theta_attr="rotary_emb_base"),
                    tie_embeddings=c.tie_word_embeddings, init_std=c.initializer_range,
                    residual="parallel" if c.use_parallel_residual else "pre", shared_parallel_norm=False)


def _neox_qkv(to_internal: bool):
    def fn(model, sd):
        H = model.config.num_attention_heads
        out = {}
        for k, v in sd.items():
            if ".attention.query_key_value." in k:
                hd = v.shape[0] // (3 * H)
                rest = v.shape[1:]
                if to_internal:
                    v = v.reshape(H, 3, hd, *rest).transpose(0, 1).reshape(3 * H * hd, *rest)
                else:
                    v = v.reshape(3, H, hd, *rest).transpose(0, 1).reshape(3 * H * hd, *rest)
            out[k] = v.contiguous()
        return out
    return fn


EXPORTS.update(define_family(
    "gpt_neox", dict(vocab_size=50432, hidden_size=6144, num_hidden_layers=44, num_attention_heads=64,
                     intermediate_size=24576, hidden_act="gelu", rotary_pct=0.25, rotary_emb_base=10000,
                     attention_dropout=0.0, hidden_dropout=0.0, classifier_dropout=0.1,
                     max_position_embeddings=2048, initializer_range=0.02, layer_norm_eps=1e-5, use_cache=True,
                     tie_word_embeddings=False, use_parallel_residual=True, rope_scaling=None, attention_bias=True),
    _neox_spec, class_prefix="GPTNeoX",
    rules=[("gpt_neox.embed_in.", "model.embed_tokens."), ("gpt_neox.final_layer_norm.", "model.norm."),
           ("gpt_neox.layers.", "model.layers."), ("embed_out.", "lm_head."),
           (".attention.query_key_value.", ".self_attn.qkv_proj."), (".attention.dense.", ".self_attn.o_proj."),
           (".mlp.dense_h_to_4h.", ".mlp.fc1."), (".mlp.dense_4h_to_h.", ".mlp.fc2.")],
    tensor_in=_neox_qkv(True), tensor_out=_neox_qkv(False), hf_keeps_fused=("qkv_proj",), layernorm_names=_LN))


# ---- gpt_j (easydel/modules/gpt_j): one shared norm, interleaved partial rotary, biased LM head ---
def _gptj_spec(c) -> ArchSpec:
    inner = c.n_inner if getattr(c, "n_inner", None) else 4 * c.n_embd
    hd = c.n_embd // c.n_head
    rope = dict(rotary_dim=hd, max_position=c.n_positions, base=10000.0, is_neox_style=False, rope_scaling=None,
                partial_rotary_factor=(c.rotary_dim or hd) / hd)
    return ArchSpec(hidden_size=c.n_embd, num_layers=c.n_layer, num_heads=c.n_head, num_kv_heads=c.n_head,
                    head_dim=hd, intermediate_size=inner, vocab_size=c.vocab_size, max_position=c.n_positions,
                    norm="layer", norm_eps=c.layer_norm_epsilon, act=c.activation_function, mlp="plain",
                    mlp_bias=True, attn_bias=False, o_bias=False, rope=rope, tie_embeddings=False,
                    init_std=c.initializer_range, residual="parallel", shared_parallel_norm=True,
                    lm_head_bias=True)


EXPORTS.update(define_family(
    "gptj", dict(vocab_size=50400, n_positions=2048, n_embd=4096, n_layer=28, n_head=16, rotary_dim=64,
                 n_inner=None, activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                 layer_norm_epsilon=1e-5, initializer_range=0.02, use_cache=True, bos_token_id=50256,
                 eos_token_id=50256, tie_word_embeddings=False),
    _gptj_spec, class_prefix="GPTJ",
    rules=[("transformer.wte.", "model.embed_tokens."), ("transformer.ln_f.", "model.norm."),
           ("transformer.h.", "model.layers."), (".ln_1.", ".input_layernorm."), (".attn.out_proj.", ".self_attn.o_proj."),
           (".attn.", ".self_attn."), (".mlp.fc_in.", ".mlp.fc1."), (".mlp.fc_out.", ".mlp.fc2.")],
    layernorm_names=_LN,
    attribute_map={"hidden_size": "n_embd", "max_position_embeddings": "n_positions",
                   "num_attention_heads": "n_head", "num_hidden_layers": "n_layer"}))


# ---- opt (easydel/modules/opt): learned positions offset by 2, ReLU MLP --------------------------
def _opt_spec(c) -> ArchSpec:
    if c.word_embed_proj_dim != c.hidden_size:
        raise NotImplementedError("OPT checkpoints with word_embed_proj_dim != hidden_size (350m) are not supported")
    if not c.do_layer_norm_before:
        raise NotImplementedError("OPT post-layer-norm variant (350m) is not supported")
    return ArchSpec(hidden_size=c.hidden_size, num_layers=c.num_hidden_layers, num_heads=c.num_attention_heads,
                    num_kv_heads=c.num_attention_heads, head_dim=c.hidden_size // c.num_attention_heads,
                    intermediate_size=c.ffn_dim, vocab_size=c.vocab_size, max_position=c.max_position_embeddings,
                    norm="layer", norm_eps=1e-5, act=c.activation_function, mlp="plain", mlp_bias=c.enable_bias,
                    attn_bias=c.enable_bias, o_bias=c.enable_bias, rope=None, pos_emb="learned",
                    learned_pos_offset=2, tie_embeddings=True, init_std=c.init_std)


EXPORTS.update(define_family(
    "opt", dict(vocab_size=50272, hidden_size=768, num_hidden_layers=12, ffn_dim=3072, max_position_embeddings=2048,
                do_layer_norm_before=True, word_embed_proj_dim=None, dropout=0.0, attention_dropout=0.0,
                num_attention_heads=12, activation_function="relu", layerdrop=0.0, init_std=0.02, use_cache=True,
                pad_token_id=1, bos_token_id=2, eos_token_id=2, enable_bias=True,
                layer_norm_elementwise_affine=True, tie_word_embeddings=True),
    _opt_spec, class_prefix="OPT",
    config_post=lambda c: setattr(c, "word_embed_proj_dim", c.word_embed_proj_dim or c.hidden_size),
    rules=[("model.decoder.final_layer_norm.", "model.norm."), ("model.decoder.", "model."),
           (".self_attn_layer_norm.", ".input_layernorm."), (".final_layer_norm.", ".post_attention_layernorm."),
           (".self_attn.out_proj.", ".self_attn.o_proj."), (".fc1.", ".mlp.fc1."), (".fc2.", ".mlp.fc2.")],
    layernorm_names=_LN))


# ---- phi (easydel/modules/phi): parallel block with one LayerNorm, partial rotary ----------------
def _phi_spec(c) -> ArchSpec:
    hd = c.hidden_size // c.num_attention_heads
    return ArchSpec(hidden_size=c.hidden_size, num_layers=c.num_hidden_layers, num_heads=c.num_attention_heads,
                    num_kv_heads=c.num_key_value_heads or c.num_attention_heads, head_dim=hd,
                    intermediate_size=c.intermediate_size, vocab_size=c.vocab_size,
                    max_position=c.max_position_embeddings, norm="layer", norm_eps=c.layer_norm_eps,
                    act=c.hidden_act, mlp="plain", mlp_bias=True, attn_bias=True, o_bias=True,
                    rope=rope_args(c, hd, partial=c.partial_rotary_factor), tie_embeddings=c.tie_word_embeddings,
                    init_std=c.initializer_range, residual="parallel", shared_parallel_norm=True,
                    lm_head_bias=True, qk_norm="layer_head" if c.qk_layernorm else None)


EXPORTS.update(define_family(
    "phi", dict(vocab_size=51200, hidden_size=2048, intermediate_size=8192, num_hidden_layers=24,
                num_attention_heads=32, num_key_value_heads=None, resid_pdrop=0.0, embd_pdrop=0.0,
                attention_dropout=0.0, hidden_act="gelu_new", max_position_embeddings=2048, initializer_range=0.02,
                layer_norm_eps=1e-5, use_cache=True, tie_word_embeddings=False, rope_theta=10000.0,
                rope_scaling=None, partial_rotary_factor=0.5, qk_layernorm=False),
    _phi_spec, rules=[("model.final_layernorm.", "model.norm."), (".self_attn.dense.", ".self_attn.o_proj.")],
    layernorm_names=_LN))


# ---- falcon (easydel/modules/falcon): three fused-QKV layouts, one or two parallel norms ----------
def _falcon_kv_heads(c) -> int:
    if c.new_decoder_architecture:
        return c.num_kv_heads or c.num_attention_heads
    return 1 if c.multi_query else c.num_attention_heads


def _falcon_spec(c) -> ArchSpec:
    if c.alibi:
        pos, rope = "alibi", None
    else:
        pos, rope = "rope", rope_args(c, c.hidden_size // c.num_attention_heads)
    two_norms = c.new_decoder_architecture and (c.num_ln_in_parallel_attn in (None, 2))
    return ArchSpec(hidden_size=c.hidden_size, num_layers=c.num_hidden_layers, num_heads=c.num_attention_heads,
                    num_kv_heads=_falcon_kv_heads(c), head_dim=c.hidden_size // c.num_attention_heads,
                    intermediate_size=c.ffn_hidden_size or 4 * c.hidden_size, vocab_size=c.vocab_size,
                    max_position=c.max_position_embeddings, norm="layer", norm_eps=c.layer_norm_epsilon,
                    act=c.activation, mlp="plain", mlp_bias=c.bias, attn_bias=c.bias, o_bias=c.bias, rope=rope,
                    pos_emb=pos, tie_embeddings=c.tie_word_embeddings, init_std=c.initializer_range,
                    residual="parallel" if (c.parallel_attn or c.new_decoder_architecture) else "pre",
                    shared_parallel_norm=not two_norms)


def _falcon_qkv(to_internal: bool):
    def fn(model, sd):
        c = model.config
        H, G = c.num_attention_heads, _falcon_kv_heads(c)
        out = {}
        for k, v in sd.items():
            if ".self_attention.query_key_value." in k and not (not c.new_decoder_architecture and c.multi_query):
                hd = v.shape[0] // (H + 2 * G)
                rest = v.shape[1:]
                qpg = H // G
                if to_internal:
                    g = v.reshape(G, qpg + 2, hd, *rest)
                    v = torch.cat([g[:, :qpg].reshape(H * hd, *rest), g[:, qpg].reshape(G * hd, *rest),
                                   g[:, qpg + 1].reshape(G * hd, *rest)], 0)
                else:
                    q = v[: H * hd].reshape(G, qpg, hd, *rest)
                    kk = v[H * hd:(H + G) * hd].reshape(G, 1, hd, *rest)
                    vv = v[(H + G) * hd:].reshape(G, 1, hd, *rest)
                    v = torch.cat([q, kk, vv], 1).reshape((H + 2 * G) * hd, *rest)
            out[k] = v.contiguous()
        return out
    return fn


def _falcon_rules(model):
    c = model.config
    rules = [("transformer.word_embeddings.", "model.embed_tokens."), ("transformer.ln_f.", "model.norm."),
             ("transformer.h.", "model.layers."), (".self_attention.query_key_value.", ".self_attn.qkv_proj."),
             (".self_attention.dense.", ".self_attn.o_proj."), (".mlp.dense_h_to_4h.", ".mlp.fc1."),
             (".mlp.dense_4h_to_h.", ".mlp.fc2.")]
    if c.new_decoder_architecture and c.num_ln_in_parallel_attn in (None, 2):
        rules += [(".ln_attn.", ".input_layernorm."), (".ln_mlp.", ".post_attention_layernorm.")]
    return rules


EXPORTS.update(define_family(
    "falcon", dict(vocab_size=65024, hidden_size=4544, num_hidden_layers=32, num_attention_heads=71,
                   num_ln_in_parallel_attn=None, layer_norm_epsilon=1e-5, initializer_range=0.02, use_cache=True,
                   hidden_dropout=0.0, attention_dropout=0.0, num_kv_heads=None, alibi=False,
                   new_decoder_architecture=False, multi_query=True, parallel_attn=True, bias=False,
                   max_position_embeddings=2048, rope_theta=10000.0, rope_scaling=None, bos_token_id=11,
                   eos_token_id=11, ffn_hidden_size=None, activation="gelu", tie_word_embeddings=True),
    _falcon_spec,
    rules=_falcon_rules,
    tensor_in=_falcon_qkv(True), tensor_out=_falcon_qkv(False), hf_keeps_fused=("qkv_proj",), layernorm_names=_LN))



# ---- mpt (easydel/modules/mosaic_mpt): ALiBi, bias-free LayerNorm and linears, fused Wqkv stored as q | k | v ------
def _mpt_spec(c) -> ArchSpec:
    ac = c.attn_config if isinstance(c.attn_config, dict) else c.attn_config.to_dict()
    return ArchSpec(hidden_size=c.d_model, num_layers=c.n_layers, num_heads=c.n_heads, num_kv_heads=c.n_heads,
                    head_dim=c.d_model // c.n_heads, intermediate_size=int(c.expansion_ratio * c.d_model),
                    vocab_size=c.vocab_size, max_position=c.max_seq_len, norm="layer", norm_bias=not c.no_bias,
                    norm_eps=c.layer_norm_epsilon, act="gelu", mlp="plain", mlp_bias=not c.no_bias,
                    attn_bias=not c.no_bias, o_bias=not c.no_bias, rope=None,
                    pos_emb="alibi" if ac.get("alibi", True) else "learned", tie_embeddings=True,
                    init_std=c.initializer_range, clip_qkv=ac.get("clip_qkv"), attn_scale=ac.get("softmax_scale"))


EXPORTS.update(define_family(
    "mpt", dict(d_model=2048, n_heads=16, n_layers=24, expansion_ratio=4, max_seq_len=2048, vocab_size=50368,
                resid_pdrop=0.0, layer_norm_epsilon=1e-5, emb_pdrop=0.0, learned_pos_emb=True,
                attn_config={"alibi": True, "clip_qkv": None, "softmax_scale": None, "qk_ln": False,
                             "attn_pdrop": 0, "alibi_bias_max": 8}, init_device="cpu", logit_scale=None,
                no_bias=True, verbose=0, embedding_fraction=1.0, norm_type="low_precision_layernorm",
                use_cache=False, initializer_range=0.02, tie_word_embeddings=True),
    _mpt_spec, class_prefix="Mpt",
    rules=[("transformer.wte.", "model.embed_tokens."), ("transformer.wpe.", "model.embed_positions."),
           ("transformer.norm_f.", "model.norm."), ("transformer.blocks.", "model.layers."),
           (".norm_1.", ".input_layernorm."), (".norm_2.", ".post_attention_layernorm."),
           (".attn.Wqkv.", ".self_attn.qkv_proj."), (".attn.out_proj.", ".self_attn.o_proj."),
           (".ffn.up_proj.", ".mlp.fc1."), (".ffn.down_proj.", ".mlp.fc2.")],
    hf_keeps_fused=("qkv_proj",), layernorm_names=_LN,
    attribute_map={"hidden_size": "d_model", "num_attention_heads": "n_heads", "num_hidden_layers": "n_layers",
                   "max_position_embeddings": "max_seq_len"}))

globals().update(EXPORTS)
__all__ = sorted(EXPORTS)
