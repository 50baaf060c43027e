"""Decoder families whose checkpoints ship with their own modelling code rather than a ``transformers`` class:
InternLM2, EXAONE-3, Grok-1 (easydel/modules/{internlm2,exaone,grok_1}). Same spec-driven decoder; the blocks below
are the name tables and the layout hooks of their checkpoints.
"""

from __future__ import annotations

import re

import torch

from ._base.families import base_spec, define_family, moe_spec

EXPORTS: dict[str, type] = {}

_LLAMA = dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
              num_attention_heads=32, num_key_value_heads=None, head_dim=None, hidden_act="silu",
              max_position_embeddings=4096, initializer_range=0.02, rms_norm_eps=1e-6, use_cache=True,
              rope_theta=10000.0, rope_scaling=None, attention_bias=False, tie_word_embeddings=False)


def _d(**kw):
    d = dict(_LLAMA)
    d.update(kw)
    return d


# ---- internlm2 (easydel/modules/internlm2): one ``wqkv`` matrix laid out per KV group as
# ---- [q_0 .. q_{g-1} | k | v] (g = query heads per KV head), MLP named w1 (gate) / w3 (up) / w2 (down) ----
def _internlm2_geometry(model):
    s = model.spec
    return s.num_heads, s.num_kv_heads, s.head_dim


def _internlm2_in(model, sd):
    hq, hkv, d = _internlm2_geometry(model)
    g = hq // hkv
    out = {}
    for k, t in sd.items():
        if ".attention.wqkv." in k:
            x = t.view(hkv, g + 2, d, *t.shape[1:])
            q = x[:, :g].reshape(hq * d, *t.shape[1:])
            kk = x[:, g].reshape(hkv * d, *t.shape[1:])
            v = x[:, g + 1].reshape(hkv * d, *t.shape[1:])
            out[k] = torch.cat([q, kk, v], 0)
        else:
            out[k] = t
    return out


def _internlm2_out(model, sd):
    hq, hkv, d = _internlm2_geometry(model)
    g = hq // hkv
    out = {}
    for k, t in sd.items():
        if ".attention.wqkv." in k:
            q, kk, v = torch.split(t, [hq * d, hkv * d, hkv * d], 0)
            x = torch.cat([q.view(hkv, g, d, *t.shape[1:]), kk.view(hkv, 1, d, *t.shape[1:]),
                           v.view(hkv, 1, d, *t.shape[1:])], 1)
            out[k] = x.reshape(-1, *t.shape[1:]).contiguous()
        else:
            out[k] = t
    return out


EXPORTS.update(define_family(
    "internlm2", _d(vocab_size=103168, bias=True, pad_token_id=0, bos_token_id=1, eos_token_id=2),
    lambda c: base_spec(c, attn_bias=getattr(c, "bias", False), o_bias=getattr(c, "bias", False)),
    class_prefix="InternLM2",
    rules=[("model.tok_embeddings.", "model.embed_tokens."), ("output.", "lm_head."),
           (".attention.wqkv.", ".self_attn.qkv_proj."), (".attention.wo.", ".self_attn.o_proj."),
           (".attention_norm.", ".input_layernorm."), (".ffn_norm.", ".post_attention_layernorm."),
           (".feed_forward.w1.", ".mlp.gate_proj."), (".feed_forward.w3.", ".mlp.up_proj."),
           (".feed_forward.w2.", ".mlp.down_proj.")],
    tensor_in=_internlm2_in, tensor_out=_internlm2_out, hf_keeps_fused=("qkv_proj",)))


# ---- exaone 3 (easydel/modules/exaone): Llama block under GPT-2 style names ----
def _exaone_post(c):
    if getattr(c, "num_hidden_layers", None) is None:
        c.num_hidden_layers = c.num_layers
    c.num_layers = c.num_hidden_layers
    c.rms_norm_eps = c.layer_norm_epsilon
    c.hidden_act = c.activation_function


EXPORTS.update(define_family(
    "exaone", dict(vocab_size=102400, hidden_size=2048, intermediate_size=14336, num_layers=32,
                   num_hidden_layers=None, num_attention_heads=32, num_key_value_heads=8, head_dim=None,
                   activation_function="silu", max_position_embeddings=2048, initializer_range=0.02,
                   layer_norm_epsilon=1e-5, use_cache=True, embed_dropout=0.0, attention_dropout=0.0,
                   rope_theta=10000.0, rope_scaling=None, tie_word_embeddings=False, bos_token_id=1, eos_token_id=2),
    lambda c: base_spec(c, norm_eps=c.layer_norm_epsilon, act=c.activation_function),
    config_post=_exaone_post, class_prefix="Exaone",
    rules=[("transformer.wte.", "model.embed_tokens."), ("transformer.ln_f.", "model.norm."),
           ("transformer.h.", "model.layers."), (".attn.attention.out_proj.", ".self_attn.o_proj."),
           (".attn.attention.", ".self_attn."), (".ln_1.", ".input_layernorm."),
           (".ln_2.", ".post_attention_layernorm."), (".mlp.c_fc_0.", ".mlp.gate_proj."),
           (".mlp.c_fc_1.", ".mlp.up_proj."), (".mlp.c_proj.", ".mlp.down_proj.")]))


# ---- grok-1 (easydel/modules/grok_1): norms before and after both branches, tanh-capped attention logits with a
# ---- fixed multiplier, GELU-gated experts (linear = gate, linear_v = up, linear_1 = down), scaled embeddings / logits
EXPORTS.update(define_family(
    "grok-1", _d(vocab_size=131072, hidden_size=6144, intermediate_size=32768, num_hidden_layers=64,
                 num_attention_heads=48, num_key_value_heads=8, attn_output_multiplier=0.08838834764831845,
                 max_attn_value=30.0, max_position_embeddings=8192, embedding_multiplier_scale=78.38367176906169,
                 output_multiplier_scale=0.5773502691896257, rms_norm_eps=1e-5, num_experts_per_tok=2,
                 num_experts=8, output_router_logits=False, router_aux_loss_coef=0.001, hidden_act="gelu"),
    lambda c: base_spec(c, sandwich_norm=True, act="gelu_new", attn_scale=c.attn_output_multiplier,
                        attn_softcap=c.max_attn_value, embedding_multiplier=c.embedding_multiplier_scale,
                        logit_scale=c.output_multiplier_scale,
                        moe=moe_spec(c, num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                     intermediate=c.intermediate_size, norm_topk=True,
                                     aux_coef=c.router_aux_loss_coef)),
    class_prefix="Grok1",
    rules=[(".attn.", ".self_attn."), (".pre_attn_norm.", ".input_layernorm."),
           (".post_attn_norm.", ".post_attn_out_layernorm."), (".pre_moe_norm.", ".pre_feedforward_layernorm."),
           (".post_moe_norm.", ".post_feedforward_layernorm."), (".moe_block.gate.", ".mlp.gate."),
           (".moe_block.experts.", ".mlp.experts."), (".linear_v.", ".up_proj."), (".linear_1.", ".down_proj."),
           (".linear.", ".gate_proj.")],
    with_classifier=False))



# ---- arctic (easydel/modules/arctic): every ``moe_layer_frequency``-th layer holds experts; there the attention
# ---- output feeds a dense hidden-sized residual MLP while the experts read the layer input in parallel ----
def _arctic_spec(c):
    n, f = c.num_hidden_layers, max(1, c.moe_layer_frequency)
    return base_spec(c, sliding_window=getattr(c, "sliding_window", None),
                     residual_mlp=bool(c.parallel_attn_mlp_res),
                     moe=moe_spec(c, num_experts=c.num_local_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.intermediate_size, norm_topk=True,
                                  layers=tuple(i for i in range(n) if (i + 1) % f == 0),
                                  aux_coef=c.router_aux_loss_coef))


EXPORTS.update(define_family(
    "arctic", _d(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=None, rms_norm_eps=1e-5, rope_theta=1e6,
                 sliding_window=None, num_experts_per_tok=1, num_local_experts=8, router_aux_loss_coef=0.001,
                 moe_layer_frequency=2, parallel_attn_mlp_res=False, moe_train_capacity_factor=1,
                 moe_eval_capacity_factor=1, moe_min_capacity=0, moe_token_dropping=True),
    _arctic_spec, class_prefix="Arctic",
    rules=[(".block_sparse_moe", ".mlp"), (".w1.", ".gate_proj."), (".w3.", ".up_proj."), (".w2.", ".down_proj.")],
    # dense layers keep their MLP one level deeper (block_sparse_moe.mlp.w1) than the experts of the sparse ones
    tensor_in=lambda model, sd: {k.replace(".block_sparse_moe.mlp.", ".block_sparse_moe."): v for k, v in sd.items()},
    tensor_out=lambda model, sd: {re.sub(r"\.block_sparse_moe\.(w[123])\.", r".block_sparse_moe.mlp.\1.", k): v
                                  for k, v in sd.items()},
    with_classifier=False))



# ---- dbrx (easydel/modules/dbrx): fused clipped ``Wqkv``, bias-free LayerNorm, 16 experts of which 4 fire, stored
# ---- as three [E * F, H] matrices (w1 gate, v1 up, w2 down with the output dimension last) ----
def _dbrx_post(c):
    a = dict(kv_n_heads=1, clip_qkv=None, rope_theta=10000.0, attn_pdrop=0.0)
    a.update(c.attn_config or {})
    f = dict(ffn_hidden_size=3584, moe_num_experts=4, moe_top_k=1, moe_jitter_eps=None, moe_loss_weight=0.01,
             moe_normalize_expert_weights=1.0, ffn_act_fn={"name": "silu"}, hidden_size=c.d_model)
    f.update(c.ffn_config or {})
    c.attn_config, c.ffn_config = a, f
    c.hidden_size, c.num_attention_heads, c.num_hidden_layers = c.d_model, c.n_heads, c.n_layers
    c.num_key_value_heads, c.max_position_embeddings = a["kv_n_heads"], c.max_seq_len
    c.rope_theta, c.intermediate_size = a["rope_theta"], f["ffn_hidden_size"]


def _dbrx_spec(c):
    f = c.ffn_config
    if f.get("moe_normalize_expert_weights") not in (None, 1, 1.0):
        raise ValueError("only L1-normalised (or un-normalised) expert weights are supported")
    return base_spec(c, norm="layer", norm_bias=False, norm_eps=1e-5, clip_qkv=c.attn_config.get("clip_qkv"),
                     act=f.get("ffn_act_fn", {}).get("name", "silu"),
                     moe=moe_spec(c, num_experts=f["moe_num_experts"], top_k=f["moe_top_k"],
                                  intermediate=f["ffn_hidden_size"],
                                  norm_topk=f.get("moe_normalize_expert_weights") is not None,
                                  aux_coef=f.get("moe_loss_weight", 0.0)))


def _dbrx_in(model, sd):
    e, fdim = model.spec.moe.num_experts, model.spec.moe.intermediate_size
    out, parts = {}, {}
    for k, t in sd.items():
        if k.endswith((".ffn.experts.mlp.w1", ".ffn.experts.mlp.v1", ".ffn.experts.mlp.w2")):
            parts.setdefault(k.rsplit(".", 1)[0], {})[k.rsplit(".", 1)[1]] = t.view(e, fdim, -1)
        else:
            out[k] = t
    for base, p in parts.items():
        pre = base[:-len("experts.mlp")]
        out[pre + "gate_up_proj.weight"] = torch.cat([p["w1"], p["v1"]], 1)
        out[pre + "down_proj.weight"] = p["w2"].transpose(1, 2)
    return out


def _dbrx_out(model, sd):
    out = {}
    for k, t in sd.items():
        if t.dim() == 3 and k.endswith(".ffn.gate_up_proj.weight"):
            f = t.shape[1] // 2
            pre = k[:-len("gate_up_proj.weight")] + "experts.mlp."
            out[pre + "w1"] = t[:, :f].reshape(-1, t.shape[2]).contiguous()
            out[pre + "v1"] = t[:, f:].reshape(-1, t.shape[2]).contiguous()
        elif t.dim() == 3 and k.endswith(".ffn.down_proj.weight"):
            out[k[:-len("down_proj.weight")] + "experts.mlp.w2"] = t.transpose(1, 2).reshape(-1, t.shape[1]).contiguous()
        else:
            out[k] = t
    return out


EXPORTS.update(define_family(
    "dbrx", dict(d_model=2048, n_heads=16, n_layers=24, max_seq_len=2048, vocab_size=32000, resid_pdrop=0.0,
                 emb_pdrop=0.0, attn_config=None, ffn_config=None, use_cache=True, initializer_range=0.02,
                 output_router_logits=False, tie_word_embeddings=False),
    _dbrx_spec, config_post=_dbrx_post, class_prefix="Dbrx",
    rules=[("transformer.wte.", "model.embed_tokens."), ("transformer.norm_f.", "model.norm."),
           ("transformer.blocks.", "model.layers."), (".norm_attn_norm.norm_1.", ".input_layernorm."),
           (".norm_attn_norm.norm_2.", ".post_attention_layernorm."),
           (".norm_attn_norm.attn.Wqkv.", ".self_attn.qkv_proj."),
           (".norm_attn_norm.attn.out_proj.", ".self_attn.o_proj."), (".ffn.router.layer.", ".mlp.gate."),
           (".ffn.", ".mlp.")],
    tensor_in=_dbrx_in, tensor_out=_dbrx_out, hf_keeps_fused=("qkv_proj", "experts"), with_classifier=False))



# ---- openelm (easydel/modules/openelm): layer-wise scaling -- the number of heads and the FFN width grow with depth;
# ---- fused ``qkv_proj`` and ``proj_1`` (gate | up) in the checkpoints, per-head QK RMSNorm, tied output layer ----
def make_divisible(v, divisor=8, min_value=None):
    divisor = divisor or 8
    min_value = min_value or divisor
    new_v = max(min_value, int(v + divisor / 2) // divisor * divisor)
    return new_v + divisor if new_v < 0.9 * v else new_v


def _linspace(a, b, n):
    return [round(a + (b - a) * i / max(n - 1, 1), 2) for i in range(n)]


def _openelm_post(c):
    n = c.num_transformer_layers
    qm = c.qkv_multipliers
    qms = [qm] * n if isinstance(qm, (int, float)) else _linspace(qm[0], qm[1], n)
    heads = [int(make_divisible(c.model_dim * m, divisor=c.head_dim * c.num_gqa_groups)) // c.head_dim for m in qms]
    c.num_query_heads, c.num_kv_heads = heads, [h // c.num_gqa_groups for h in heads]
    fm = c.ffn_multipliers
    c.ffn_multipliers = [fm] * n if isinstance(fm, (int, float)) else \
        (_linspace(fm[0], fm[1], n) if len(fm) == 2 else list(fm))
    c.hidden_size, c.num_hidden_layers, c.max_position_embeddings = c.model_dim, n, c.max_context_length
    c.num_attention_heads, c.num_key_value_heads = max(heads), max(c.num_kv_heads)
    c.intermediate_size = max(int(make_divisible(m * c.model_dim, c.ffn_dim_divisor)) for m in c.ffn_multipliers)
    c.rope_theta = c.rope_freq_constant


def _openelm_spec(c):
    per = tuple(dict(num_heads=q, num_kv_heads=k,
                     intermediate_size=int(make_divisible(m * c.model_dim, c.ffn_dim_divisor)))
                for q, k, m in zip(c.num_query_heads, c.num_kv_heads, c.ffn_multipliers))
    return base_spec(c, norm_eps=1e-6, act=c.activation_fn_name, mlp="gated" if c.ffn_with_glu else "plain",
                     qk_norm="rms_head" if c.normalize_qk_projections else None,
                     tie_embeddings=c.share_input_output_layers, per_layer=per)


EXPORTS.update(define_family(
    "openelm", dict(vocab_size=32000, max_context_length=2048, num_transformer_layers=12, model_dim=2048, head_dim=128,
                    qkv_multipliers=1.0, num_gqa_groups=1, ffn_multipliers=4.0, ffn_with_glu=True, ffn_dim_divisor=256,
                    activation_fn_name="swish", normalization_layer_name="rms_norm", normalize_qk_projections=False,
                    share_input_output_layers=False, rope_freq_constant=10000, rope_max_length=4096,
                    initializer_range=0.02, use_cache=True, rope_scaling=None),
    _openelm_spec, config_post=_openelm_post, class_prefix="OpenELM",
    rules=[("transformer.token_embeddings.", "model.embed_tokens."), ("transformer.norm.", "model.norm."),
           ("transformer.layers.", "model.layers."), (".attn.out_proj.", ".self_attn.o_proj."),
           (".attn.", ".self_attn."), (".attn_norm.", ".input_layernorm."),
           (".ffn_norm.", ".post_attention_layernorm."), (".ffn.proj_1.", ".mlp.gate_up_proj."),
           (".ffn.proj_2.", ".mlp.down_proj.")],
    hf_keeps_fused=("qkv_proj", "gate_up_proj"), with_classifier=False))



# ---- gidd (easydel/modules/gidd): a bidirectional diffusion language model. (1 + w) RMSNorm, squared-ReLU MLP without
# ---- gate, residual branches scaled by ``resid_scale``; q and k are L2-normalised over the whole projection and each
# ---- head has a learned temperature ``qk_scale`` (initialised to 2 log(max positions)) instead of 1 / sqrt(d) ----
def _gidd_spec(c):
    import math as _m

    qk = bool(c.use_qk_norm)
    return base_spec(c, norm_offset=1.0, mlp="plain", act="relu2", mlp_bias=c.mlp_bias, causal=False,
                     residual_multiplier=c.resid_scale, qk_norm="l2_full" if qk else None, qk_norm_eps=c.qk_norm_eps,
                     attn_scale=1.0 if qk else None,
                     attn_head_scale_init=2 * _m.log(c.max_position_embeddings) if qk else None)


_GIDD = define_family(
    "gidd", _d(vocab_size=131072, hidden_size=768, intermediate_size=3072, num_hidden_layers=12,
               num_attention_heads=12, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=10000.0,
               init_scale=0.4, emb_init_scale=0.1, head_init_scale=0.0, resid_scale=4.0, use_qk_norm=True,
               qk_norm_eps=1e-6, mlp_bias=False, tie_word_embeddings=False),
    _gidd_spec, class_prefix="Gidd",
    rules=[(".mlp.up_proj.", ".mlp.fc1."), (".mlp.down_proj.", ".mlp.fc2."), (".self_attn.qk_scale", ".self_attn.head_scale")],
    tensor_in=lambda model, sd: {k: (v.reshape(-1) if k.endswith(".self_attn.qk_scale") else v) for k, v in sd.items()},
    tensor_out=lambda model, sd: {k: (v.reshape(1, 1, -1, 1) if k.endswith(".self_attn.qk_scale") else v)
                                  for k, v in sd.items()},
    with_classifier=False)


class GiddForDiffusionLM(_GIDD["GiddForCausalLM"]):
    """Denoising head: logits for every position from the bidirectional backbone; the loss is cross-entropy at the
    positions whose label is not ``ignore_index`` (the noised tokens), without the next-token shift."""

    loss_type = "ForDiffusionLM"

    def _compute_task_loss(self, labels, loss_config, loss_scale, call, loss_kwargs):
        from ..infra.loss_utils import LossMetrics

        call = {k: v for k, v in call.items() if k not in ("noise_mask", "log_snr")}
        out = self(**call)
        lg = out.logits.float()
        loss = torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), labels.reshape(-1),
                                                 ignore_index=loss_config.ignore_index)
        return out, LossMetrics(loss=loss * loss_scale)


from ..infra.factory import TaskType as _TaskType, register_module as _register_module  # noqa: E402

GiddForDiffusionLM = _register_module(_TaskType.DIFFUSION_LM, config=_GIDD["GiddConfig"], model_type="gidd")(
    GiddForDiffusionLM)
_GIDD["GiddForDiffusionLM"] = GiddForDiffusionLM
EXPORTS.update(_GIDD)



# ---- xerxes (easydel/modules/xerxes): Gemma-2 style block (norms before and after both branches, scaled embeddings,
# ---- every ``window_pattern``-th layer global, the others sliding) with optional per-head QK norm and experts; with
# ---- QK norm on and neither experts nor ``xe_mlpnorm`` it degenerates to the plain pre-norm block ----
def _xerxes_plain(c) -> bool:
    return bool(c.xe_kvnorm and not c.xe_moe and not c.xe_mlpnorm)


def _xerxes_spec(c):
    import math as _m

    n = c.num_hidden_layers
    types = None
    if c.window_pattern:
        types = tuple("sliding" if (i + 1) % c.window_pattern else "full" for i in range(n))
    moe = None
    if c.xe_moe:
        moe = moe_spec(c, num_experts=c.num_local_experts, top_k=c.num_experts_per_tok,
                       intermediate=c.intermediate_size, norm_topk=True)
    return base_spec(c, sandwich_norm=not _xerxes_plain(c), qk_norm="rms_head" if c.xe_kvnorm else None,
                     act="silu" if c.swish_run else "gelu_new", layer_types=types, sliding_window=c.sliding_window,
                     embed_scale=1.0 if (c.xe_kvnorm and not c.xe_mlpnorm) else _m.sqrt(c.hidden_size), moe=moe,
                     tie_embeddings=getattr(c, "tie_word_embeddings", False))


def _sandwich_rules(model):
    plain = not model.spec.sandwich_norm if hasattr(model, "spec") else False
    return [] if plain else [(".post_attention_layernorm.", ".post_attn_out_layernorm.")]


EXPORTS.update(define_family(
    "xerxes", _d(vocab_size=256128, hidden_size=4096, intermediate_size=16384, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=16384,
                 rms_norm_eps=1e-6, num_local_experts=8, num_experts_per_tok=2, swish_run=False, xe_moe=False,
                 xe_kvnorm=False, xe_mlpnorm=False, window_pattern=None, sliding_window=4096),
    _xerxes_spec, class_prefix="Xerxes", rules=_sandwich_rules))


# ---- xerxes2 (easydel/modules/xerxes2): latent (MLA) attention inside the same four-norm block, Qwen-style experts ----
def _xerxes2_spec(c):
    qk = c.qk_nope_head_dim + c.qk_rope_head_dim
    moe = None
    if c.num_experts:
        only = set(c.mlp_only_layers or [])
        step = c.decoder_sparse_step or 1
        layers = tuple(i for i in range(c.num_hidden_layers) if i not in only and (i + 1) % step == 0)
        moe = moe_spec(c, num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                       intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob, layers=layers,
                       aux_coef=c.router_aux_loss_coef)
    from .families import rope_args as _rope_args

    return base_spec(c, head_dim=c.qk_rope_head_dim, rope=_rope_args(c, c.qk_rope_head_dim), sandwich_norm=True,
                     mla=dict(q_lora_rank=c.q_lora_dim, kv_lora_rank=c.kv_lora_dim,
                              qk_nope_head_dim=c.qk_nope_head_dim, qk_rope_head_dim=c.qk_rope_head_dim,
                              v_head_dim=c.vhead_dim, scale=qk ** -0.5, rope_interleave=False), moe=moe)


_X2 = _d(vocab_size=256128, hidden_size=4096, intermediate_size=16384, moe_intermediate_size=8192,
         decoder_sparse_step=1, num_experts=8, num_experts_per_tok=2, norm_topk_prob=False,
         output_router_logits=False, router_aux_loss_coef=0.001, num_hidden_layers=32, num_attention_heads=32,
         max_position_embeddings=16384, rms_norm_eps=1e-6, q_lora_dim=1536, kv_lora_dim=512, qk_rope_head_dim=64,
         qk_nope_head_dim=128, vhead_dim=128, mlp_only_layers=None)
_X2.pop("head_dim", None)
EXPORTS.update(define_family("xerxes2", _X2, _xerxes2_spec, class_prefix="Xerxes2",
                             rules=[(".post_attention_layernorm.", ".post_attn_out_layernorm.")],
                             with_classifier=False))

globals().update(EXPORTS)
__all__ = sorted(EXPORTS)
