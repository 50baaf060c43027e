"""Gemma-4 text model (easydel/modules/gemma4/modeling_gemma4.py:1002-2826).

What sets the architecture apart from the spec-driven decoder families, and why it has a module of its own:

* sliding layers use ``head_dim``; full-attention layers use ``global_head_dim`` and, with ``attention_k_eq_v``, fewer
  KV heads (``num_global_key_value_heads``) and no value projection: the value is the un-normalised key projection;
* queries and keys get a learned per-head RMSNorm, values a weightless one, and the softmax scale is 1;
* full-attention layers rotate only the first ``partial_rotary_factor`` of the frequency pairs ("proportional" rotary:
  the remaining pairs have frequency zero), sliding layers use the plain rotary with their own base;
* the last ``num_kv_shared_layers`` layers own no keys / values: each reads those of the last earlier layer of its
  own type (and may have a double-width MLP);
* every layer can receive a per-layer input: a second embedding table ``[vocab, L * P]`` plus a projection of the
  token embedding, gated into the residual stream after the MLP;
* an optional expert block runs in parallel with the dense MLP (router = weightless RMSNorm, learned scale,
  softmax, renormalised top-k, per-expert scale), each branch with its own post-norm;
* each layer's output is multiplied by a stored scalar.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.loss_utils import LossConfig, LossMetrics
from ...infra.modeling_outputs import BaseModelOutput, CausalLMOutput
from ...layers.norms import RMSNorm
from ...ops import functional as F
from ...ops import reference as R
from ...ops.grouped import moe_ffn

_ROPE_DEFAULT = {
    "sliding_attention": {"rope_type": "default", "rope_theta": 10_000.0},
    "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1_000_000.0},
}


@register_config("gemma4_text")
class Gemma4TextConfig(EasyDeLBaseConfig):
    model_type = "gemma4_text"
    hf_config_keys = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                      "num_key_value_heads", "head_dim", "hidden_activation", "max_position_embeddings",
                      "rms_norm_eps", "rope_parameters", "attention_bias", "sliding_window", "layer_types",
                      "final_logit_softcapping", "vocab_size_per_layer_input", "hidden_size_per_layer_input",
                      "num_global_key_value_heads", "global_head_dim", "attention_k_eq_v", "num_kv_shared_layers",
                      "enable_moe_block", "use_double_wide_mlp", "num_experts", "top_k_experts",
                      "moe_intermediate_size", "tie_word_embeddings")

    def __init__(self, vocab_size=262_144, hidden_size=2304, intermediate_size=9216, num_hidden_layers=30,
                 num_attention_heads=8, num_key_value_heads=4, head_dim=256, hidden_activation="gelu_pytorch_tanh",
                 max_position_embeddings=131_072, initializer_range=0.02, rms_norm_eps=1e-6, rope_parameters=None,
                 attention_bias=False, sliding_window=512, layer_types=None, final_logit_softcapping=None,
                 vocab_size_per_layer_input=262_144, hidden_size_per_layer_input=256,
                 num_global_key_value_heads=None, global_head_dim=512, attention_k_eq_v=False,
                 num_kv_shared_layers=0, enable_moe_block=False, use_double_wide_mlp=False, num_experts=None,
                 top_k_experts=None, moe_intermediate_size=None, pad_token_id=0, eos_token_id=1, bos_token_id=2,
                 tie_word_embeddings=True, **kw):
        self.vocab_size, self.hidden_size, self.intermediate_size = vocab_size, hidden_size, intermediate_size
        self.num_hidden_layers, self.num_attention_heads = num_hidden_layers, num_attention_heads
        self.num_key_value_heads, self.head_dim = num_key_value_heads, head_dim
        self.hidden_activation, self.max_position_embeddings = hidden_activation, max_position_embeddings
        self.initializer_range, self.rms_norm_eps, self.attention_bias = initializer_range, rms_norm_eps, attention_bias
        self.sliding_window, self.final_logit_softcapping = sliding_window, final_logit_softcapping
        if layer_types is None:      # five sliding layers, then a full one
            layer_types = ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(num_hidden_layers)]
        layer_types = list(layer_types)
        layer_types[-1] = "full_attention"
        self.layer_types = layer_types
        self.rope_parameters = rope_parameters or {k: dict(v) for k, v in _ROPE_DEFAULT.items()}
        self.vocab_size_per_layer_input = vocab_size_per_layer_input
        self.hidden_size_per_layer_input = hidden_size_per_layer_input
        self.num_global_key_value_heads, self.global_head_dim = num_global_key_value_heads, global_head_dim
        self.attention_k_eq_v, self.num_kv_shared_layers = attention_k_eq_v, num_kv_shared_layers
        self.enable_moe_block, self.use_double_wide_mlp = enable_moe_block, use_double_wide_mlp
        self.num_experts, self.top_k_experts, self.moe_intermediate_size = num_experts, top_k_experts, \
            moe_intermediate_size
        super().__init__(pad_token_id=pad_token_id, eos_token_id=eos_token_id, bos_token_id=bos_token_id,
                         tie_word_embeddings=tie_word_embeddings, **kw)

    # --- per-layer geometry ------------------------------------------------------------------------------------
    def first_shared_layer(self) -> int:
        return self.num_hidden_layers - (self.num_kv_shared_layers or 0)

    def kv_donor(self, i: int) -> int | None:
        """The layer whose keys / values layer ``i`` reads, or ``None`` when it owns them."""
        first = self.first_shared_layer()
        if not (i >= first > 0):
            return None
        prev = self.layer_types[:first]
        return len(prev) - 1 - prev[::-1].index(self.layer_types[i])

    def layer_geometry(self, i: int) -> tuple[int, int, bool]:
        """``(head_dim, kv_heads, k_eq_v)`` of layer ``i``."""
        sliding = self.layer_types[i] == "sliding_attention"
        hd = self.head_dim if sliding or not self.global_head_dim else self.global_head_dim
        alt = bool(self.attention_k_eq_v) and not sliding
        return hd, (self.num_global_key_value_heads if alt else self.num_key_value_heads), alt


class Gemma4Cache:
    """Dense decode cache with per-layer head geometry; layers that borrow keys / values hold nothing."""

    def __init__(self, config: Gemma4TextConfig, batch: int, max_len: int, dtype, device):
        self.length, self.max_len = 0, max_len
        self.k, self.v = {}, {}
        for i in range(config.num_hidden_layers):
            if config.kv_donor(i) is None:
                hd, hk, _ = config.layer_geometry(i)
                self.k[i] = torch.zeros(batch, max_len, hk, hd, dtype=dtype, device=device)
                self.v[i] = torch.zeros(batch, max_len, hk, hd, dtype=dtype, device=device)

    def seq_len(self) -> int:
        return self.length

    def advance(self, n: int) -> None:
        self.length += n

    def reorder(self, index: torch.Tensor) -> None:
        for d in (self.k, self.v):
            for i in d:
                d[i] = d[i].index_select(0, index)


class _Rotary(nn.Module):
    def __init__(self, config: Gemma4TextConfig):
        super().__init__()
        for lt in set(config.layer_types):
            p = config.rope_parameters[lt]
            prop = p.get("rope_type", "default") == "proportional"
            hd = config.global_head_dim if (prop and lt == "full_attention") else config.head_dim
            n_rot = int(p.get("partial_rotary_factor", 1.0) * hd // 2) if prop else hd // 2
            inv = 1.0 / (p["rope_theta"] ** (torch.arange(0, 2 * n_rot, 2, dtype=torch.float32) / hd))
            inv = torch.cat([inv, torch.zeros(hd // 2 - n_rot)]) / p.get("factor", 1.0)
            self.register_buffer(f"{lt}_inv_freq", inv, persistent=False)

    def forward(self, positions: torch.Tensor, layer_type: str):
        ang = positions[..., None].float() * getattr(self, f"{layer_type}_inv_freq").to(positions.device)
        return ang.cos()[:, :, None], ang.sin()[:, :, None]          # [B, T, 1, hd/2]


class _Attention(nn.Module):
    def __init__(self, c: Gemma4TextConfig, i: int, dtype):
        super().__init__()
        self.layer_idx, self.layer_type = i, c.layer_types[i]
        self.sliding_window = c.sliding_window if self.layer_type == "sliding_attention" else None
        self.head_dim, self.kv_heads, self.k_eq_v = c.layer_geometry(i)
        self.heads, self.donor = c.num_attention_heads, c.kv_donor(i)
        self.eps = c.rms_norm_eps
        H, b = c.hidden_size, c.attention_bias
        self.q_proj = nn.Linear(H, self.heads * self.head_dim, bias=b, dtype=dtype)
        self.q_norm = RMSNorm(self.head_dim, c.rms_norm_eps, dtype)
        self.o_proj = nn.Linear(self.heads * self.head_dim, H, bias=b, dtype=dtype)
        if self.donor is None:
            self.k_proj = nn.Linear(H, self.kv_heads * self.head_dim, bias=b, dtype=dtype)
            self.k_norm = RMSNorm(self.head_dim, c.rms_norm_eps, dtype)
            if not self.k_eq_v:
                self.v_proj = nn.Linear(H, self.kv_heads * self.head_dim, bias=b, dtype=dtype)

    def keys_values(self, x, cos, sin):
        B, T, _ = x.shape
        k_raw = F.linear(x, self.k_proj.weight, self.k_proj.bias).view(B, T, self.kv_heads, self.head_dim)
        v = k_raw if self.k_eq_v else F.linear(x, self.v_proj.weight, self.v_proj.bias).view(k_raw.shape)
        k = R.rotate(self.k_norm(k_raw).float(), cos, sin).to(x.dtype)
        v = (v.float() * torch.rsqrt(v.float().pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        return k, v

    def forward(self, x, cos, sin, shared: dict, segment_ids=None, cache: Gemma4Cache | None = None, meta=None):
        B, T, _ = x.shape
        q = F.linear(x, self.q_proj.weight, self.q_proj.bias).view(B, T, self.heads, self.head_dim)
        q = R.rotate(self.q_norm(q).float(), cos, sin).to(x.dtype)
        if self.donor is None:
            k, v = self.keys_values(x, cos, sin)
            if cache is not None:
                s, e = cache.length, cache.length + T
                if e > cache.max_len:
                    raise ValueError(f"KV cache overflow: {e} > {cache.max_len}")
                cache.k[self.layer_idx][:, s:e] = k
                cache.v[self.layer_idx][:, s:e] = v
                k, v = cache.k[self.layer_idx][:, :e], cache.v[self.layer_idx][:, :e]
            shared[self.layer_idx] = (k, v)
        else:
            k, v = shared[self.donor]
        if cache is not None and meta is not None and meta.get("kv_segment_ids") is not None:
            seg_k = meta["kv_segment_ids"][:, :k.shape[1]]
            o = R.attention(q, k, v, causal=True, scale=1.0, segment_ids=seg_k[:, -T:], kv_segment_ids=seg_k,
                            sliding_window=self.sliding_window)
        else:
            if cache is not None and B > 1:
                k, v = k.contiguous(), v.contiguous()
            o = F.attention(q, k, v, causal=True, scale=1.0, segment_ids=None if cache is not None else segment_ids,
                            sliding_window=self.sliding_window)
        return F.linear(o.reshape(B, T, -1), self.o_proj.weight, self.o_proj.bias)


class _MLP(nn.Module):
    def __init__(self, c: Gemma4TextConfig, i: int, dtype):
        super().__init__()
        wide = c.use_double_wide_mlp and c.kv_donor(i) is not None
        inner = c.intermediate_size * (2 if wide else 1)
        self.act = c.hidden_activation
        self.gate_proj = nn.Linear(c.hidden_size, inner, bias=False, dtype=dtype)
        self.up_proj = nn.Linear(c.hidden_size, inner, bias=False, dtype=dtype)
        self.down_proj = nn.Linear(inner, c.hidden_size, bias=False, dtype=dtype)

    def forward(self, x):
        gu = torch.cat([F.linear(x, self.gate_proj.weight), F.linear(x, self.up_proj.weight)], -1)
        return F.linear(F.gated_act(gu, self.act), self.down_proj.weight)


class _Router(nn.Module):
    def __init__(self, c: Gemma4TextConfig, dtype):
        super().__init__()
        self.eps, self.top_k, self.root = c.rms_norm_eps, c.top_k_experts, c.hidden_size ** -0.5
        self.proj = nn.Linear(c.hidden_size, c.num_experts, bias=False, dtype=dtype)
        self.scale = nn.Parameter(torch.ones(c.hidden_size, dtype=dtype))
        self.per_expert_scale = nn.Parameter(torch.ones(c.num_experts, dtype=dtype))

    def forward(self, x):
        xf = x.float()
        h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.scale * self.root
        probs = torch.softmax(F.linear(h, self.proj.weight).float(), -1)
        w, idx = torch.topk(probs, self.top_k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        return probs, (w * self.per_expert_scale.float()[idx]).to(x.dtype), idx


class _Experts(nn.Module):
    def __init__(self, c: Gemma4TextConfig, dtype):
        super().__init__()
        E, H, I = c.num_experts, c.hidden_size, c.moe_intermediate_size
        self.act = c.hidden_activation
        self.gate_up_proj = nn.Parameter(torch.randn(E, 2 * I, H, dtype=dtype) * c.initializer_range)
        self.down_proj = nn.Parameter(torch.randn(E, H, I, dtype=dtype) * c.initializer_range)

    def forward(self, x, idx, w):
        return moe_ffn(x, self.gate_up_proj, self.down_proj, w, idx, act=self.act)


class _Layer(nn.Module):
    def __init__(self, c: Gemma4TextConfig, i: int, dtype):
        super().__init__()
        H, eps = c.hidden_size, c.rms_norm_eps
        self.self_attn = _Attention(c, i, dtype)
        self.mlp = _MLP(c, i, dtype)
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                  "post_feedforward_layernorm"):
            setattr(self, n, RMSNorm(H, eps, dtype))
        self.register_buffer("layer_scalar", torch.ones(1, dtype=dtype))
        self.per_layer = bool(c.hidden_size_per_layer_input)
        if self.per_layer:
            self.act = c.hidden_activation
            self.per_layer_input_gate = nn.Linear(H, c.hidden_size_per_layer_input, bias=False, dtype=dtype)
            self.per_layer_projection = nn.Linear(c.hidden_size_per_layer_input, H, bias=False, dtype=dtype)
            self.post_per_layer_input_norm = RMSNorm(H, eps, dtype)
        self.moe = bool(c.enable_moe_block)
        if self.moe:
            self.router = _Router(c, dtype)
            self.experts = _Experts(c, dtype)
            for n in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                setattr(self, n, RMSNorm(H, eps, dtype))

    def forward(self, x, per_layer_input, cos, sin, shared, segment_ids, cache, meta):
        x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), cos, sin, shared, segment_ids,
                                                             cache, meta))
        h = self.mlp(self.pre_feedforward_layernorm(x))
        router_probs = None
        if self.moe:
            flat = x.reshape(-1, x.shape[-1])
            router_probs, w, idx = self.router(flat)
            h2 = self.experts(self.pre_feedforward_layernorm_2(flat), idx, w).view(x.shape)
            h = self.post_feedforward_layernorm_1(h) + self.post_feedforward_layernorm_2(h2)
        x = x + self.post_feedforward_layernorm(h)
        if self.per_layer:
            g = R.ACT2FN[self.act](F.linear(x, self.per_layer_input_gate.weight)) * per_layer_input
            x = x + self.post_per_layer_input_norm(F.linear(g, self.per_layer_projection.weight))
        return x * self.layer_scalar, router_probs


class Gemma4TextModel(EasyDeLBaseModule):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self._build(config, self.param_dtype)

    def _build(self, c, dt):
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dt)
        nn.init.normal_(self.embed_tokens.weight, std=c.initializer_range)
        self.layers = nn.ModuleList([_Layer(c, i, dt) for i in range(c.num_hidden_layers)])
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps, dt)
        self.rotary = _Rotary(c)
        P = c.hidden_size_per_layer_input
        if P:
            self.embed_tokens_per_layer = nn.Embedding(c.vocab_size_per_layer_input, c.num_hidden_layers * P, dtype=dt)
            nn.init.normal_(self.embed_tokens_per_layer.weight, std=c.initializer_range)
            self.per_layer_model_projection = nn.Linear(c.hidden_size, c.num_hidden_layers * P, bias=False, dtype=dt)
            self.per_layer_projection_norm = RMSNorm(P, c.rms_norm_eps, dt)

    def embed(self, input_ids):
        return self.embed_tokens(input_ids) * torch.tensor(self.config.hidden_size ** 0.5,
                                                           dtype=self.embed_tokens.weight.dtype)

    def per_layer_inputs(self, input_ids, inputs_embeds, given=None):
        c = self.config
        P, L = c.hidden_size_per_layer_input, c.num_hidden_layers
        if not P:
            return None
        proj = F.linear(inputs_embeds, self.per_layer_model_projection.weight) * c.hidden_size ** -0.5
        proj = self.per_layer_projection_norm(proj.view(*inputs_embeds.shape[:-1], L, P))
        if given is None and input_ids is not None:
            given = (self.embed_tokens_per_layer(input_ids) * torch.tensor(P ** 0.5, dtype=proj.dtype)).view(
                *input_ids.shape, L, P)
        if given is None:
            return proj
        return (proj + given) * 2.0 ** -0.5

    def forward(self, input_ids=None, inputs_embeds=None, position_ids=None, attention_mask=None, segment_ids=None,
                past_key_values: Gemma4Cache | None = None, cache_metadata=None, per_layer_inputs=None,
                output_hidden_states=False, **_):
        c = self.config
        if inputs_embeds is None:
            inputs_embeds = self.embed(input_ids)
        B, T, _ = inputs_embeds.shape
        pli = self.per_layer_inputs(input_ids, inputs_embeds, per_layer_inputs)
        if position_ids is None:
            start = past_key_values.length if past_key_values is not None else 0
            position_ids = torch.arange(start, start + T, device=inputs_embeds.device)[None].expand(B, T)
        if segment_ids is None and attention_mask is not None and past_key_values is None and \
                not bool(attention_mask.all()):
            segment_ids = attention_mask.to(torch.int32)
        rope = {lt: self.rotary(position_ids, lt) for lt in set(c.layer_types)}
        x, shared, hs, probs = inputs_embeds, {}, [], []
        for i, layer in enumerate(self.layers):
            if output_hidden_states:
                hs.append(x)
            cos, sin = rope[c.layer_types[i]]
            x, p = layer(x, None if pli is None else pli[:, :, i], cos, sin, shared, segment_ids, past_key_values,
                         cache_metadata)
            if p is not None:
                probs.append(p)
        x = self.norm(x)
        if output_hidden_states:
            hs.append(x)
        out = BaseModelOutput(last_hidden_state=x, hidden_states=tuple(hs) if output_hidden_states else None,
                              past_key_values=past_key_values)
        out.router_probs = tuple(probs) if probs else None
        return out

    def init_cache(self, batch_size, max_length, dtype=None, device=None, **_):
        p = self.embed_tokens.weight if hasattr(self, "embed_tokens") else self.model.embed_tokens.weight
        return Gemma4Cache(self.config, batch_size, max_length, dtype or p.dtype, device or p.device)


register_module(TaskType.BASE_MODULE, config=Gemma4TextConfig, model_type="gemma4_text")(Gemma4TextModel)


@register_module(TaskType.CAUSAL_LM, config=Gemma4TextConfig, model_type="gemma4_text")
class Gemma4ForCausalLM(EasyDeLBaseModule):
    loss_type = "ForCausalLM"
    hf_keeps_fused = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.model = Gemma4TextModel(config, dtype, param_dtype, precision, rngs)
        if not config.tie_word_embeddings:
            self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False, dtype=self.param_dtype)

    init_cache = Gemma4TextModel.init_cache

    def can_generate(self):
        return True

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def lm_head_weight(self):
        return self.model.embed_tokens.weight if self.config.tie_word_embeddings else self.lm_head.weight

    def lm_head_bias(self):
        return None

    def apply_lm_head(self, h):
        logits = F.linear(h, self.lm_head_weight())
        cap = self.config.final_logit_softcapping
        if cap:
            logits = (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)
        return logits

    def forward(self, input_ids=None, inputs_embeds=None, apply_lm_head: bool = True, **kw):
        out = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds, **kw)
        logits = self.apply_lm_head(out.last_hidden_state) if apply_lm_head else None
        res = CausalLMOutput(logits=logits, last_hidden_state=out.last_hidden_state, hidden_states=out.hidden_states,
                             past_key_values=out.past_key_values)
        res.router_probs = out.router_probs
        return res

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        call = {k: v for k, v in call.items() if k != "labels"}
        out = self(**call)
        lg = out.logits[:, :-1].float()
        tgt = labels[:, 1:]
        mask = call.get("attention_mask")
        if mask is not None:
            tgt = tgt.masked_fill(mask[:, 1:] == 0, loss_config.ignore_index)
        loss = torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), tgt.reshape(-1),
                                                 ignore_index=loss_config.ignore_index)
        return out, LossMetrics(loss=loss * loss_scale)

    # ------------------------------------------------------------------ checkpoint names
    # Own names equal the published ones except that layers which borrow keys / values keep no key / value tensors.
    def hf_rename_in(self, sd):
        own = set(self.state_dict().keys())
        return {k: v for k, v in sd.items() if k in own}

    def hf_rename_out(self, sd):
        return dict(sd)


# =====================================================================================================================
# Vision tower and the multimodal model (easydel/modules/gemma4/modeling_gemma4.py:239-1000, 2826-3367)
# =====================================================================================================================
from .._base.families import _Renamer  # noqa: E402
from .._base.vlm import OUTER_RULES, VLMConfig, VLMForConditionalGeneration  # noqa: E402


@register_config("gemma4_vision")
class Gemma4VisionConfig(EasyDeLBaseConfig):
    model_type = "gemma4_vision"
    hf_config_keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                      "num_key_value_heads", "head_dim", "hidden_activation", "rms_norm_eps", "rope_parameters",
                      "pooling_kernel_size", "patch_size", "position_embedding_size", "use_clipped_linears",
                      "standardize")

    def __init__(self, hidden_size=768, intermediate_size=3072, num_hidden_layers=16, num_attention_heads=12,
                 num_key_value_heads=12, head_dim=64, hidden_activation="gelu_pytorch_tanh", rms_norm_eps=1e-6,
                 max_position_embeddings=131_072, rope_parameters=None, pooling_kernel_size=3, patch_size=16,
                 position_embedding_size=10 * 1024, use_clipped_linears=False, standardize=False,
                 initializer_range=0.02, **kw):
        self.hidden_size, self.intermediate_size, self.num_hidden_layers = hidden_size, intermediate_size, \
            num_hidden_layers
        self.num_attention_heads, self.num_key_value_heads, self.head_dim = num_attention_heads, \
            num_key_value_heads, head_dim
        self.hidden_activation, self.rms_norm_eps = hidden_activation, rms_norm_eps
        self.max_position_embeddings = max_position_embeddings
        self.rope_parameters = rope_parameters or {"rope_type": "default", "rope_theta": 100.0}
        self.pooling_kernel_size, self.patch_size = pooling_kernel_size, patch_size
        self.position_embedding_size, self.use_clipped_linears = position_embedding_size, use_clipped_linears
        self.standardize, self.initializer_range = standardize, initializer_range
        super().__init__(**kw)


@register_config("gemma4")
class Gemma4Config(VLMConfig):
    model_type = "gemma4"
    vision_default, text_default = "gemma4_vision", "gemma4_text"

    def __init__(self, text_config=None, vision_config=None, audio_config=None, boi_token_id=255_999,
                 eoi_token_id=258_882, image_token_id=258_880, video_token_id=258_884, boa_token_id=256_000,
                 eoa_token_index=258_883, audio_token_id=258_881, **kw):
        if isinstance(vision_config, dict):
            vision_config = dict(vision_config, model_type="gemma4_vision")
        if isinstance(text_config, dict):
            text_config = dict(text_config, model_type="gemma4_text")
        kw.setdefault("tie_word_embeddings", True)
        kw = self._init_parts(vision_config, text_config, image_token_id, kw)
        self.audio_config = audio_config          # an opaque payload kept for round trips, as in the reference
        self.boi_token_id, self.eoi_token_id, self.image_token_id = boi_token_id, eoi_token_id, image_token_id
        self.video_token_id, self.boa_token_id, self.eoa_token_index = video_token_id, boa_token_id, eoa_token_index
        self.audio_token_id = audio_token_id
        super().__init__(**kw)


class _ClippableLinear(nn.Module):
    """Bias-free linear whose input and output may be clamped to stored ranges (quantisation-aware checkpoints)."""

    def __init__(self, c: Gemma4VisionConfig, d_in, d_out, dtype):
        super().__init__()
        self.clip = c.use_clipped_linears
        self.linear = nn.Linear(d_in, d_out, bias=False, dtype=dtype)
        if self.clip:
            for n, v in (("input_min", -float("inf")), ("input_max", float("inf")), ("output_min", -float("inf")),
                         ("output_max", float("inf"))):
                self.register_buffer(n, torch.tensor(v))

    def forward(self, x):
        if self.clip:
            x = torch.clamp(x, self.input_min, self.input_max)
        y = F.linear(x, self.linear.weight)
        return torch.clamp(y, self.output_min, self.output_max) if self.clip else y


class _VisionAttention(nn.Module):
    def __init__(self, c: Gemma4VisionConfig, dtype):
        super().__init__()
        H, hd = c.hidden_size, c.head_dim
        self.heads, self.kv_heads, self.head_dim, self.eps = c.num_attention_heads, c.num_key_value_heads, hd, \
            c.rms_norm_eps
        self.q_proj = _ClippableLinear(c, H, self.heads * hd, dtype)
        self.k_proj = _ClippableLinear(c, H, self.kv_heads * hd, dtype)
        self.v_proj = _ClippableLinear(c, H, self.kv_heads * hd, dtype)
        self.o_proj = _ClippableLinear(c, self.heads * hd, H, dtype)
        self.q_norm, self.k_norm = RMSNorm(hd, c.rms_norm_eps, dtype), RMSNorm(hd, c.rms_norm_eps, dtype)

    @staticmethod
    def _rope2d(x, cos, sin):
        # the head splits in two halves: the first turns with the patch column, the second with the row
        h = x.shape[-1] // 2
        q = h // 2
        a = R.rotate(x[..., :h].float(), cos[..., :q], sin[..., :q])
        b = R.rotate(x[..., h:].float(), cos[..., q:], sin[..., q:])
        return torch.cat([a, b], -1).to(x.dtype)

    def forward(self, x, cos, sin, seg):
        B, T, _ = x.shape
        q = self._rope2d(self.q_norm(self.q_proj(x).view(B, T, self.heads, self.head_dim)), cos, sin)
        k = self._rope2d(self.k_norm(self.k_proj(x).view(B, T, self.kv_heads, self.head_dim)), cos, sin)
        v = self.v_proj(x).view(B, T, self.kv_heads, self.head_dim)
        v = (v.float() * torch.rsqrt(v.float().pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        o = F.attention(q, k, v, causal=False, scale=1.0, segment_ids=seg)
        return self.o_proj(o.reshape(B, T, -1))


class _VisionMLP(nn.Module):
    def __init__(self, c: Gemma4VisionConfig, dtype):
        super().__init__()
        self.act = c.hidden_activation
        self.gate_proj = _ClippableLinear(c, c.hidden_size, c.intermediate_size, dtype)
        self.up_proj = _ClippableLinear(c, c.hidden_size, c.intermediate_size, dtype)
        self.down_proj = _ClippableLinear(c, c.intermediate_size, c.hidden_size, dtype)

    def forward(self, x):
        return self.down_proj(R.ACT2FN[self.act](self.gate_proj(x)) * self.up_proj(x))


class _VisionLayer(nn.Module):
    def __init__(self, c: Gemma4VisionConfig, dtype):
        super().__init__()
        self.self_attn, self.mlp = _VisionAttention(c, dtype), _VisionMLP(c, dtype)
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                  "post_feedforward_layernorm"):
            setattr(self, n, RMSNorm(c.hidden_size, c.rms_norm_eps, dtype))

    def forward(self, x, cos, sin, seg):
        x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), cos, sin, seg))
        return x + self.post_feedforward_layernorm(self.mlp(self.pre_feedforward_layernorm(x)))


class Gemma4VisionModel(nn.Module):
    """``pixel_values`` ``[B, patches, 3 * P * P]`` in ``[0, 1]`` and ``pixel_position_ids`` ``[B, patches, 2]`` (x, y;
    ``-1`` marks padding) -> soft tokens ``[n_valid, hidden]``: the patches are encoded, averaged over
    ``k x k`` neighbourhoods of the grid (``k = pooling_kernel_size``) and scaled by ``sqrt(hidden)``."""

    def __init__(self, c: Gemma4VisionConfig, dtype):
        super().__init__()
        self.cfg = c
        self.patch_embedder = nn.Module()
        self.patch_embedder.input_proj = nn.Linear(3 * c.patch_size ** 2, c.hidden_size, bias=False, dtype=dtype)
        self.patch_embedder.position_embedding_table = nn.Parameter(
            torch.randn(2, c.position_embedding_size, c.hidden_size, dtype=dtype) * c.initializer_range)
        self.encoder = nn.Module()
        self.encoder.layers = nn.ModuleList([_VisionLayer(c, dtype) for _ in range(c.num_hidden_layers)])
        sp = c.head_dim // 2
        self.register_buffer("inv_freq", 1.0 / (c.rope_parameters["rope_theta"] ** (
            torch.arange(0, sp, 2, dtype=torch.float32) / sp)), persistent=False)
        if c.standardize:
            self.register_buffer("std_bias", torch.zeros(c.hidden_size))
            self.register_buffer("std_scale", torch.ones(c.hidden_size))

    def forward(self, pixel_values, pixel_position_ids):
        c = self.cfg
        pad = (pixel_position_ids == -1).all(-1)
        pos = pixel_position_ids.clamp(min=0)
        tab = self.patch_embedder.position_embedding_table
        w = self.patch_embedder.input_proj.weight
        x = F.linear((2 * (pixel_values - 0.5)).to(w.dtype), w)
        pe = tab[0][pos[..., 0]] + tab[1][pos[..., 1]]
        x = x + torch.where(pad[..., None], torch.zeros_like(pe), pe)
        ang = pixel_position_ids[..., None].float() * self.inv_freq            # [B, T, 2, hd/4]
        cos, sin = ang.cos().flatten(-2)[:, :, None], ang.sin().flatten(-2)[:, :, None]
        seg = (~pad).to(torch.int32)
        for layer in self.encoder.layers:
            x = layer(x, cos, sin, seg)
        x = x.masked_fill(pad[..., None], 0.0)
        T = x.shape[1]
        length = T // (c.pooling_kernel_size ** 2)
        valid = ~pad
        if length != T:
            k = int((T // length) ** 0.5)
            if k * k * length != T:
                raise ValueError(f"cannot pool {T} patches to {length} soft tokens")
            max_x = pos[..., 0].max(-1, keepdim=True)[0] + 1
            cell = torch.div(pos, k, rounding_mode="floor")
            cell = cell[..., 0] + (max_x // k) * cell[..., 1]
            wts = torch.nn.functional.one_hot(cell.long(), length).float() / (k * k)
            x = (wts.transpose(1, 2) @ x.float()).to(x.dtype)
            valid = ~(wts == 0).all(1)
        x = (x * c.hidden_size ** 0.5)[valid]
        if c.standardize:
            x = (x - self.std_bias) * self.std_scale
        return x


class _MultimodalEmbedder(nn.Module):
    def __init__(self, d_in, d_out, eps, dtype):
        super().__init__()
        self.eps = eps
        self.embedding_projection = nn.Linear(d_in, d_out, bias=False, dtype=dtype)

    def forward(self, x):
        xf = x.float()
        return F.linear((xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype),
                        self.embedding_projection.weight)


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Gemma4Config, model_type="gemma4")
class Gemma4ForConditionalGeneration(VLMForConditionalGeneration):
    """Image soft tokens replace the ``image_token_id`` embeddings. The per-layer inputs are looked up with the
    placeholder positions set to the padding id, before the merge."""

    outer_rules = [*OUTER_RULES, ("model.embed_vision.", "embed_vision.")]
    ignored_prefixes = ("model.audio_tower.", "model.embed_audio.")
    image_kwargs = ("image_position_ids",)

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.vision_tower = Gemma4VisionModel(config.vision_config, self.param_dtype)
        self.embed_vision = _MultimodalEmbedder(config.vision_config.hidden_size, config.text_config.hidden_size,
                                                config.vision_config.rms_norm_eps, self.param_dtype)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)

    def _vision_renamer(self):
        return _Renamer([])

    def get_image_features(self, pixel_values, image_position_ids=None, **kw):
        if image_position_ids is None:
            raise ValueError("Gemma-4 needs image_position_ids ([B, patches, 2]) with pixel_values")
        return self.embed_vision(self.vision_tower(pixel_values, image_position_ids))

    def _mm_mask(self, input_ids):
        c = self.config
        return (input_ids == c.image_token_id) | (input_ids == c.video_token_id) | (input_ids == c.audio_token_id)

    def embed_text(self, input_ids):
        ids = input_ids.masked_fill(self._mm_mask(input_ids), self.config.text_config.pad_token_id or 0)
        return self.language_model.model.embed(ids)

    def _per_layer(self, input_ids):
        tm = self.language_model.model
        if not self.config.text_config.hidden_size_per_layer_input:
            return None
        ids = input_ids.masked_fill(self._mm_mask(input_ids), self.config.text_config.pad_token_id or 0)
        P = self.config.text_config.hidden_size_per_layer_input
        e = tm.embed_tokens_per_layer(ids) * torch.tensor(P ** 0.5, dtype=tm.embed_tokens_per_layer.weight.dtype)
        return e.view(*ids.shape, self.config.text_config.num_hidden_layers, P)

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                past_key_values=None, image_features=None, **kw):
        extra = {k: kw.pop(k) for k in self.image_kwargs if k in kw}
        if inputs_embeds is None:
            first = past_key_values is None or past_key_values.seq_len() == 0
            inputs_embeds = self.merge_embeddings(input_ids, pixel_values if first else None,
                                                  image_features if first else None, **extra)
            kw.setdefault("per_layer_inputs", self._per_layer(input_ids))
        return self.language_model(inputs_embeds=inputs_embeds, attention_mask=attention_mask,
                                   position_ids=position_ids, past_key_values=past_key_values, **kw)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        call = dict(call)
        ids = call.pop("input_ids")
        extra = {k: call.pop(k) for k in self.image_kwargs if k in call}
        call["inputs_embeds"] = self.merge_embeddings(ids, call.pop("pixel_values", None),
                                                      call.pop("image_features", None), **extra)
        call["per_layer_inputs"] = self._per_layer(ids)
        labels = labels.masked_fill(self._mm_mask(ids), loss_config.ignore_index)
        return self.language_model._compute_task_loss(labels, loss_config, loss_scale, call, loss_kwargs)
