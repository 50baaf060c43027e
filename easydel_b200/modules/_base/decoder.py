"""Spec-driven decoder-only transformer shared by the model families.

Each family (``modules/<name>``) maps its Hugging Face style config onto an :class:`ArchSpec`
(normalisation kind, MLP kind, positional scheme, QK-norm, sliding-window layout, MoE layout,
soft-caps, tying, residual topology...) and registers thin subclasses of the classes here. The
layer loop keeps the residual stream and the not-yet-added branch output as a pair so that every
residual add is fused into the following RMSNorm kernel.

Reference structure being covered: ``LlamaDecoderLayer`` / ``LlamaModel`` / ``LlamaForCausalLM``
(easydel/modules/llama/modeling_llama.py:165-564) and the task heads in
easydel/modules/_base/causal_lm_module.py:84-627.
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass, field

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from ...infra.base_module import EasyDeLBaseModule
from ...infra.loss_utils import (LossConfig, LossMetrics, ForSequenceClassificationLoss,
                                 auxiliary_load_balancing_loss_func, causal_lm_loss_from_hidden)
from ...infra.modeling_outputs import (BaseModelOutput, CausalLMOutput, MoeCausalLMOutput, MoeModelOutput,
                                       SequenceClassifierOutput)
from ...layers.attention import Attention
from ...layers.embeddings import Embed
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import GatedMLP, PlainMLP
from ...layers.moe import MoEBlock
from ...layers.norms import LayerNorm, RMSNorm
from ...ops import functional as F


@dataclass
class MoESpec:
    num_experts: int
    top_k: int
    intermediate_size: int
    norm_topk_prob: bool = True
    scoring: str = "softmax"
    routed_scaling_factor: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    use_score_bias: bool = False
    router_bias: bool = False
    shared_intermediate_size: int = 0
    shared_gate: bool = False
    layers: tuple[int, ...] | None = None   # None = every layer
    aux_loss_coef: float = 0.0
    expert_init_std: float = 0.01
    expert_bias: bool = False         # per-expert biases on both expert projections (GPT-OSS)
    expert_act: str | None = None     # gated activation of the experts when it differs from the dense MLP's
    scale_input: bool = False         # routing score applied to the experts' input (Llama-4)
    router_jitter_eps: float = 0.01   # margin of the sparsemixer routing (Phi-3.5-MoE)
    routing_strategy: str | None = None          # top_k | top_k_ndiv | switch | expert_choice | hash; None = by scoring
    capacity_factor: float | None = None         # None = dropless
    load_balancing_strategy: str = "standard"    # standard | switch_transformer | expert_choice | none
    lbl_coef: float | None = None                # per-block load-balancing loss (added to the training loss)
    rzl_coef: float | None = None                # per-block router z-loss


def _first_set(*values):
    return next((v for v in values if v is not None), None)


@dataclass
class ArchSpec:
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position: int = 4096
    norm: str = "rms"                 # rms | layer
    norm_eps: float = 1e-6
    norm_offset: float = 0.0          # Gemma: weights stored as (w - 1)
    norm_bias: bool = True            # LayerNorm only
    act: str = "silu"
    mlp: str = "gated"                # gated | plain
    mlp_bias: bool = False
    attn_bias: bool = False
    o_bias: bool = False
    qk_norm: str | None = None
    rope: dict | None = None          # kwargs of layers.rotary.get_rope minus head_size; None = no RoPE
    rope_local: dict | None = None    # separate table for sliding layers (Gemma3)
    pos_emb: str = "rope"             # rope | learned | alibi | none
    learned_pos_offset: int = 0
    tie_embeddings: bool = False
    embed_scale: float | None = None
    logit_softcap: float = 0.0
    attn_softcap: float = 0.0
    attn_scale: float | None = None
    sliding_window: int | None = None
    layer_types: tuple[str, ...] | None = None  # per layer: "full" | "sliding" | "nope" (full, no rope)
    residual: str = "pre"             # pre | parallel | post (norm applied to the branch output, OLMo2)
    sandwich_norm: bool = False       # extra norms after attention / MLP outputs (Gemma2/3)
    shared_parallel_norm: bool = True  # parallel residual with one norm (GPT-J, Phi) vs two (NeoX)
    use_sinks: bool = False
    moe: MoESpec | None = None
    lm_head_bias: bool = False
    final_norm: bool = True
    embed_layernorm: bool = False
    init_std: float = 0.02
    clip_qkv: float | None = None
    logit_scale: float | None = None  # Cohere / Granite style multiplier on logits
    residual_multiplier: float | None = None
    embedding_multiplier: float | None = None
    mla: dict | None = None           # kwargs of layers.mla.MLAttention: latent attention instead of MHA / GQA
    linear_attn: dict | None = None   # kwargs of layers.linear_attention.GatedDeltaNet for layers of type "linear"
    attn_output_gate: bool = False    # sigmoid gate on the attention output, emitted by the query projection
    attn_chunk_size: int | None = None  # block-diagonal attention on the rotary layers of a rope / nope mix (Llama-4)
    attn_temp_tuning: tuple[float, float] | None = None  # (attn_scale, floor_scale) on the layers without rotary
    qk_norm_rope_only: bool = False   # QK norm only on layers that rotate
    causal: bool = True               # False: bidirectional blocks (diffusion language models)
    attn_head_scale_init: float | None = None  # learned per-head query multiplier (GIDD)
    qk_norm_eps: float | None = None  # epsilon of the QK norm when it differs from the block norms'
    per_layer: tuple | None = None    # one dict of field overrides per layer (OpenELM scales heads / FFN by depth)
    lightning: dict | None = None     # kwargs of layers.lightning_attention.LightningAttention for "lightning" layers
    normed_residual: dict | None = None  # MiniMax: the branch input (after the norm) is the residual, combined as
                                      # alpha * normed + beta * branch; keys attn / lightning / mlp -> (alpha, beta)
    ssm_branch: dict | None = None    # kwargs of layers.ssm_branch.SSDMixer: a Mamba-2 mixer beside attention (Falcon-H1)
    branch_multipliers: tuple[float, float, float] = (1.0, 1.0, 1.0)  # attention input, attention output, SSM output
    mlp_multipliers: tuple[float, float] = (1.0, 1.0)                  # gate pre-activation, MLP output
    residual_mlp: bool = False        # Arctic: MoE layers add a dense hidden-sized MLP branch after attention while
                                      # the experts read the layer input (norm of x, not of x + attention)


def _norm(spec: ArchSpec, dtype) -> nn.Module:
    if spec.norm == "rms":
        return RMSNorm(spec.hidden_size, spec.norm_eps, dtype, offset=spec.norm_offset)
    if spec.norm == "layer_noparam":
        return LayerNorm(spec.hidden_size, spec.norm_eps if spec.norm_eps > 1e-6 else 1e-5, dtype=dtype,
                         elementwise_affine=False)
    return LayerNorm(spec.hidden_size, spec.norm_eps, bias=spec.norm_bias, dtype=dtype)


def _resolve(x):
    """Tensor-parallel products may arrive as pending reductions (see ``parallel.tp.PendingReduce``)."""
    return x.resolve() if hasattr(x, "resolve") else x


def _tp_of(config) -> tuple[int, int, tp.Any]:
    mesh = config.mesh
    if mesh.tp > 1:
        return mesh.tp, mesh.axis_index("tp"), mesh.get_group("tp")
    return 1, 0, None


def _ep_of(config) -> tuple[int, int, tp.Any]:
    mesh = config.mesh
    if mesh.ep > 1:
        return mesh.ep, mesh.axis_index("ep"), mesh.get_group("ep")
    return 1, 0, None


class DecoderLayer(nn.Module):
    def __init__(self, config, spec: ArchSpec, layer_idx: int, dtype):
        super().__init__()
        self.spec, self.layer_idx = spec, layer_idx
        tp_size, tp_rank, tp_group = _tp_of(config)
        ltype = spec.layer_types[layer_idx] if spec.layer_types else ("sliding" if spec.sliding_window else "full")
        window = spec.sliding_window if ltype == "sliding" else None
        rope = spec.rope if spec.pos_emb == "rope" else None
        if ltype == "sliding" and spec.rope_local is not None:
            rope = spec.rope_local
        if ltype == "nope":
            rope = None
        self.is_linear = ltype in ("linear", "lightning", "kda")
        self.ltype = ltype
        if ltype == "lightning":
            from ...layers.lightning_attention import LightningAttention

            self.self_attn = LightningAttention(spec.hidden_size, spec.num_heads, spec.head_dim, spec.num_layers,
                                                act=spec.act, layer_idx=layer_idx,
                                                dtype=dtype, init_std=spec.init_std, **spec.lightning)
        elif ltype == "kda":
            from ...layers.linear_attention import KimiDeltaAttention

            self.linear_attn = KimiDeltaAttention(spec.hidden_size, layer_idx=layer_idx, dtype=dtype,
                                                  init_std=spec.init_std, norm_eps=spec.norm_eps, **spec.linear_attn)
        elif self.is_linear:
            from ...layers.linear_attention import GatedDeltaNet

            self.linear_attn = GatedDeltaNet(spec.hidden_size, layer_idx=layer_idx, dtype=dtype,
                                             init_std=spec.init_std, norm_eps=spec.norm_eps, **spec.linear_attn)
        elif spec.mla is not None:
            from ...layers.mla import MLAttention

            self.self_attn = MLAttention(spec.hidden_size, spec.num_heads, rope=spec.rope, norm_eps=spec.norm_eps,
                                         bias=spec.attn_bias, layer_idx=layer_idx, dtype=dtype,
                                         init_std=spec.init_std, tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group,
                                         **spec.mla)
        else:
            self.self_attn = self._mha(spec, layer_idx, dtype, rope, window, tp_size, tp_rank, tp_group)
        if spec.ssm_branch is not None:
            from ...layers.ssm_branch import SSDMixer

            self.mamba = SSDMixer(spec.hidden_size, layer_idx=layer_idx, dtype=dtype, init_std=spec.init_std,
                                  norm_eps=spec.norm_eps, **spec.ssm_branch)
        moe = spec.moe
        self.is_moe = moe is not None and (moe.layers is None or layer_idx in moe.layers)
        self._build_mlp(config, spec, layer_idx, dtype, tp_size, tp_rank, tp_group)
        if spec.mlp_multipliers != (1.0, 1.0) and hasattr(self.mlp, "gate_multiplier"):
            self.mlp.gate_multiplier, self.mlp.down_multiplier = spec.mlp_multipliers
        fused = spec.norm == "rms" and spec.residual == "pre" and not spec.sandwich_norm \
            and spec.residual_multiplier is None
        if fused and tp_size > 1 and spec.mla is None and not self.is_linear and spec.ssm_branch is None \
                and spec.normed_residual is None:
            # both branch outputs feed a fused add+norm: let it also do the tensor-parallel sum
            self.self_attn.o_proj.defer_reduce = True
            if not self.is_moe:
                (self.mlp.down_proj if hasattr(self.mlp, "down_proj") else self.mlp.fc2).defer_reduce = True

    @staticmethod
    def _mha(spec, layer_idx, dtype, rope, window, tp_size, tp_rank, tp_group):
        qk_norm = spec.qk_norm if (rope is not None or not spec.qk_norm_rope_only) else None
        return Attention(
            spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim, layer_idx=layer_idx,
            bias=spec.attn_bias, o_bias=spec.o_bias, qk_norm=qk_norm,
            qk_norm_eps=spec.qk_norm_eps if spec.qk_norm_eps is not None else spec.norm_eps, rope=rope,
            causal=spec.causal, head_scale_init=spec.attn_head_scale_init,
            chunk_size=spec.attn_chunk_size if rope is not None else None,
            temp_tuning=spec.attn_temp_tuning if rope is None else None,
            sliding_window=window, softcap=spec.attn_softcap, scale=spec.attn_scale, use_sinks=spec.use_sinks,
            use_alibi=spec.pos_emb == "alibi", clip_qkv=spec.clip_qkv, dtype=dtype, init_std=spec.init_std,
            tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group, qk_norm_offset=spec.norm_offset,
            output_gate=spec.attn_output_gate)

    def _build_mlp(self, config, spec, layer_idx, dtype, tp_size, tp_rank, tp_group):
        moe = spec.moe
        if self.is_moe:
            ep_size, ep_rank, ep_group = _ep_of(config)
            self.mlp = MoEBlock(spec.hidden_size, moe.intermediate_size, moe.num_experts, moe.top_k,
                                act=moe.expert_act or spec.act, expert_bias=moe.expert_bias,
                                scale_input=moe.scale_input, router_jitter_eps=moe.router_jitter_eps,
                                routing_strategy=getattr(config, "moe_routing_strategy", None) or moe.routing_strategy,
                                capacity_factor=getattr(config, "moe_capacity_factor", None) or moe.capacity_factor,
                                load_balancing_strategy=getattr(config, "moe_load_balancing_strategy", None)
                                or moe.load_balancing_strategy,
                                lbl_coef=_first_set(getattr(config, "moe_lbl_coef", None), moe.lbl_coef),
                                rzl_coef=_first_set(getattr(config, "moe_rzl_coef", None), moe.rzl_coef),
                                norm_topk_prob=moe.norm_topk_prob, scoring=moe.scoring,
                                routed_scaling_factor=moe.routed_scaling_factor, n_group=moe.n_group,
                                topk_group=moe.topk_group, use_score_bias=moe.use_score_bias,
                                router_bias=moe.router_bias, shared_intermediate_size=moe.shared_intermediate_size,
                                shared_gate=moe.shared_gate, dtype=dtype, init_std=spec.init_std,
                                expert_init_std=moe.expert_init_std, ep_size=ep_size, ep_rank=ep_rank,
                                ep_group=ep_group, tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group,
                                expert_tensor_mode=bool(getattr(config, "use_expert_tensor_mode", False)))
        elif spec.mlp == "gated":
            self.mlp = GatedMLP(spec.hidden_size, spec.intermediate_size, spec.act, spec.mlp_bias, dtype,
                                spec.init_std, tp_size, tp_rank, tp_group)
        else:
            self.mlp = PlainMLP(spec.hidden_size, spec.intermediate_size, spec.act, spec.mlp_bias, dtype,
                                spec.init_std, tp_size, tp_rank, tp_group)
        self.has_residual_mlp = bool(spec.residual_mlp and self.is_moe)
        if self.has_residual_mlp:
            self.residual_layernorm = _norm(spec, dtype)
            self.residual_mlp = GatedMLP(spec.hidden_size, spec.hidden_size, spec.act, False, dtype, spec.init_std,
                                         tp_size, tp_rank, tp_group)
        if spec.residual == "post":
            self.post_attention_layernorm = _norm(spec, dtype)
            self.post_feedforward_layernorm = _norm(spec, dtype)
        else:
            self.input_layernorm = _norm(spec, dtype)
            if (spec.residual == "pre" and not spec.sandwich_norm) or \
                    (spec.residual == "parallel" and not spec.shared_parallel_norm):
                self.post_attention_layernorm = _norm(spec, dtype)
            if spec.sandwich_norm:
                self.post_attn_out_layernorm = _norm(spec, dtype)
                self.pre_feedforward_layernorm = _norm(spec, dtype)
                self.post_feedforward_layernorm = _norm(spec, dtype)

    # The pair (x, pending) means the residual stream is x + pending; `pending` is folded in by the
    # next fused add+norm. Returns (x, pending, router_logits).
    def _mix(self, h, positions, segment_ids, cache_view, attn_meta):
        state = None
        if cache_view is not None and (self.ltype == "lightning" or self.is_linear or self.spec.ssm_branch is not None):
            state = cache_view.linear_state
        try:
            if self.ltype == "lightning":
                return self.self_attn(h, segment_ids=segment_ids, state=state)
            if self.is_linear:
                return self.linear_attn(h, segment_ids=segment_ids, state=state)
            if self.spec.ssm_branch is not None:
                a_in, a_out, s_out = self.spec.branch_multipliers
                m = self.mamba(h, segment_ids=segment_ids, state=state)
                a = self.self_attn(h * a_in if a_in != 1.0 else h, positions, segment_ids=segment_ids,
                                   cache_view=cache_view, attn_meta=attn_meta)
                return m * s_out + a * a_out
        finally:
            if hasattr(state, "commit"):      # serving: write the scheduled sequences' states back to their slots
                state.commit()
        return self.self_attn(h, positions, segment_ids=segment_ids, cache_view=cache_view, attn_meta=attn_meta)

    def forward(self, x, pending, positions, segment_ids=None, cache_view=None, attn_meta=None):
        spec = self.spec
        rl = None
        fused = spec.norm == "rms" and spec.residual == "pre" and not spec.sandwich_norm \
            and spec.residual_multiplier is None and not self.has_residual_mlp
        if spec.normed_residual is not None:
            if pending is not None:
                x = x + _resolve(pending)
            nr = spec.normed_residual
            a_a, b_a = nr["lightning" if self.ltype == "lightning" else "attn"]
            a_m, b_m = nr["mlp"]
            h = self.input_layernorm(x)
            x = h * a_a + self._mix(h, positions, segment_ids, cache_view, attn_meta) * b_a
            h = self.post_attention_layernorm(x)
            m = self.mlp(h)
            if self.is_moe:
                m, rl = m
            return h * a_m + m * b_m, None, rl
        if self.has_residual_mlp:
            if pending is not None:
                x = x + _resolve(pending)
            x1 = x + self._mix(self.input_layernorm(x), positions, segment_ids, cache_view, attn_meta)
            r = x1 + self.residual_mlp(self.residual_layernorm(x1))
            m, rl = self.mlp(self.post_attention_layernorm(x))
            return r + m, None, rl
        if fused:
            if pending is None:
                h = self.input_layernorm(x)
            else:
                h, x = self.input_layernorm.forward_with_residual(pending, x)
            a = self._mix(h, positions, segment_ids, cache_view, attn_meta)
            h, x = self.post_attention_layernorm.forward_with_residual(a, x)
            m = self.mlp(h)
            if self.is_moe:
                m, rl = m
            return x, m, rl
        if pending is not None:
            x = x + _resolve(pending)
        rm = spec.residual_multiplier or 1.0
        if spec.residual == "parallel":
            h = self.input_layernorm(x)
            a = self._mix(h, positions, segment_ids, cache_view, attn_meta)
            h2 = h if spec.shared_parallel_norm else self.post_attention_layernorm(x)
            m = self.mlp(h2)
            if self.is_moe:
                m, rl = m
            return x + a + m, None, rl
        if spec.residual == "post":
            a = self._mix(x, positions, segment_ids, cache_view, attn_meta)
            x = x + self.post_attention_layernorm(a)
            m = self.mlp(x)
            if self.is_moe:
                m, rl = m
            return x + self.post_feedforward_layernorm(m), None, rl
        h = self.input_layernorm(x)
        a = self._mix(h, positions, segment_ids, cache_view, attn_meta)
        if spec.sandwich_norm:
            a = self.post_attn_out_layernorm(a)
        x = x + a * rm
        h = (self.pre_feedforward_layernorm if spec.sandwich_norm else self.post_attention_layernorm)(x)
        m = self.mlp(h)
        if self.is_moe:
            m, rl = m
        if spec.sandwich_norm:
            m = self.post_feedforward_layernorm(m)
        return x + m * rm, None, rl


class DecoderModel(EasyDeLBaseModule):
    """Embedding -> N decoder layers -> final norm."""

    spec_fn: tp.Callable[[tp.Any], ArchSpec] | None = None

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        spec = type(self).spec_fn(config)
        self.spec = spec
        pd = self.param_dtype
        self.embed_tokens = Embed(spec.vocab_size, spec.hidden_size, pd, spec.init_std,
                                  getattr(config, "pad_token_id", None) if False else None)
        if spec.pos_emb == "learned":
            self.embed_positions = Embed(spec.max_position + spec.learned_pos_offset, spec.hidden_size, pd,
                                         spec.init_std)
        if spec.embed_layernorm:
            self.embed_layernorm = _norm(spec, pd)
        import dataclasses

        def layer_spec(i):
            if spec.per_layer is None:
                return spec
            return dataclasses.replace(spec, per_layer=None, **spec.per_layer[i])

        self.layers = nn.ModuleList([DecoderLayer(config, layer_spec(i), i, pd) for i in range(spec.num_layers)])
        if spec.final_norm:
            self.norm = _norm(spec, pd)
        self._setup_sequence_parallel(config)
        self._setup_context_parallel(config)

    #: process group over which the sequence dimension of a batch is sharded (``attn_mechanism="ring"``), or None
    cp_group = None
    cp_layout = "zigzag"

    def _setup_context_parallel(self, config) -> None:
        """``attn_mechanism="ring"`` on a mesh whose ``sp`` axis is larger than one: every rank of the ``sp`` group
        runs the layers on its slice of the sequence and the attention layers see the whole sequence's keys
        (parallel.context_parallel). The reference selects its ring attention the same way
        (easydel/operations/kernels/ring_attention.py:84-260) with the batch sharded ``P(("dp", "fsdp"), "sp")``."""
        mesh = getattr(config, "mesh", None)
        mech = str(getattr(getattr(config, "attn_mechanism", None), "value", getattr(config, "attn_mechanism", "")))
        if mesh is None or getattr(mesh, "sp", 1) <= 1 or mech != "ring":
            return
        self.cp_group = mesh.get_group("sp")
        self.cp_layout = getattr(config, "ring_attention_layout", None) or "zigzag"
        impl = getattr(config, "ring_attention_impl", None) or "auto"
        for layer in self.layers:
            attn = getattr(layer, "self_attn", None)
            if attn is not None and hasattr(attn, "cp_group"):
                attn.cp_group, attn.cp_layout, attn.cp_impl = self.cp_group, self.cp_layout, impl

    def _setup_sequence_parallel(self, config) -> None:
        """Dense attention + MLP stacks can keep the residual stream sharded by rows over the tensor-parallel
        group between their linears (all-gather -> GEMM into the column layers, GEMM -> reduce-scatter out of the
        row layers). The state object is shared with every tensor-parallel linear of the layers."""
        from ...layers.linears import ParallelLinear
        from ...parallel.tp import SequenceParallelState

        self.sp = SequenceParallelState()
        tp_size, _, tp_group = _tp_of(config)
        self._sp_group = tp_group
        plain = all(not l.is_moe and not l.is_linear and l.ltype != "lightning" and l.spec.mla is None
                    and l.spec.ssm_branch is None and l.spec.normed_residual is None for l in self.layers)
        self.sp_capable = bool(tp_size > 1 and plain and getattr(config, "tp_sequence_parallel", True))
        if self.sp_capable:
            for m in self.layers.modules():
                if isinstance(m, ParallelLinear) and m.tp_size > 1:
                    m.sp_state = self.sp

    def get_input_embeddings(self):
        return self.embed_tokens

    #: set by ``EasyDeLState.init_tx`` when the decoder layers are parameter-sharded (``parallel.fsdp``)
    fsdp_layers = None

    def _run_layer(self, layer, x, pending, positions, segment_ids, cache_view, attn_meta, policy):
        if self.fsdp_layers is not None and cache_view is None:
            # the layer's weights are gathered for the call; under autograd the layer is a recompute unit
            return self.fsdp_layers.run(layer.layer_idx, layer, x, _resolve(pending), positions, segment_ids,
                                        self.remat_policy())
        if policy and self.training and torch.is_grad_enabled() and cache_view is None:
            # recompute unit under the configured save policy (full recompute, saved dots, saved names ...)
            from ...ops import remat

            return remat.recompute_unit(lambda a, b, c, d: layer(a, b, c, d, None, None), self.remat_policy(),
                                        (x, _resolve(pending), positions, segment_ids))
        return layer(x, pending, positions, segment_ids, cache_view, attn_meta)

    def forward(self, input_ids: torch.Tensor | None = None, attention_mask: torch.Tensor | None = None,
                position_ids: torch.Tensor | None = None, segment_ids: torch.Tensor | None = None,
                inputs_embeds: torch.Tensor | None = None, past_key_values=None, cache_metadata=None,
                output_hidden_states: bool = False, output_router_logits: bool = False,
                deepstack_embeds: tp.Sequence[torch.Tensor] | None = None, sequence_parallel: bool = False, **_):
        """``deepstack_embeds[i]`` ``[B, T, H]`` (zeros outside image positions) is added to the residual stream
        after layer ``i`` (Qwen3-VL feeds intermediate vision features to the first decoder layers).

        ``sequence_parallel``: the caller takes ``last_hidden_state`` as this rank's row shard ``[1, B*T/tp, H]``
        (rows of the flattened ``[B*T]`` token axis) when ``self.sp.active`` is set on return."""
        spec = self.spec
        if inputs_embeds is None:
            if input_ids.dim() == 1:
                input_ids = input_ids[None]
            x = self.embed_tokens(input_ids)
        else:
            x = inputs_embeds
        B, T = x.shape[:2]
        if x.dtype != self.dtype and x.is_floating_point():
            x = x.to(self.dtype)
        if spec.embed_scale is not None:
            x = x * torch.tensor(spec.embed_scale, dtype=x.dtype, device=x.device)
        if spec.embedding_multiplier is not None:
            x = x * spec.embedding_multiplier
        if position_ids is None:
            start = 0
            if past_key_values is not None and hasattr(past_key_values, "seq_len"):
                start = past_key_values.seq_len()
            if segment_ids is not None:
                position_ids = _positions_from_segments(segment_ids)
            elif attention_mask is not None and past_key_values is None:
                position_ids = (attention_mask.long().cumsum(-1) - 1).clamp_min(0)
            else:
                position_ids = torch.arange(start, start + T, device=x.device)[None].expand(B, T)
        if position_ids.dim() == 1:
            position_ids = position_ids[None].expand(B, T)
        if segment_ids is None and attention_mask is not None and past_key_values is None and T > 1:
            # padding -> segment 0 (isolated), real tokens -> segment 1
            if not bool(attention_mask.all()):
                segment_ids = attention_mask.to(torch.int32)
        if spec.pos_emb == "learned":
            x = x + self.embed_positions(position_ids + spec.learned_pos_offset)
        if spec.embed_layernorm:
            x = self.embed_layernorm(x)
        use_sp = bool(sequence_parallel and self.sp_capable and past_key_values is None and not output_hidden_states
                      and deepstack_embeds is None and (B * T) % self.config.mesh.tp == 0)
        if use_sp:
            from ...parallel import tp as tpar

            self.sp.begin(self._sp_group, B, T)
            x = tpar.shard_rows(self.sp, x)
        else:
            self.sp.end()
        policy = self.gradient_checkpointing_policy() not in ("", "everything_saveable")
        pending = None
        all_hidden = [] if output_hidden_states else None
        router_logits = []
        for i, layer in enumerate(self.layers):
            if output_hidden_states:
                pending = _resolve(pending)
                all_hidden.append(x if pending is None else x + pending)
            view = past_key_values.view(i) if past_key_values is not None else None
            x, pending, rl = self._run_layer(layer, x, pending, position_ids, segment_ids, view, cache_metadata,
                                             policy)
            if rl is not None:
                router_logits.append(rl)
            if deepstack_embeds is not None and i < len(deepstack_embeds):
                x = x + deepstack_embeds[i].to(x.dtype)
        if spec.final_norm:
            if pending is not None and spec.norm == "rms":
                x, _ = self.norm.forward_with_residual(pending, x)
            else:
                x = self.norm(x if pending is None else x + _resolve(pending))
        elif pending is not None:
            x = x + _resolve(pending)
        if output_hidden_states:
            all_hidden.append(x)
        cls = MoeModelOutput if spec.moe is not None else BaseModelOutput
        kw = dict(last_hidden_state=x, hidden_states=tuple(all_hidden) if all_hidden else None,
                  past_key_values=past_key_values)
        if spec.moe is not None:
            kw["router_logits"] = tuple(router_logits) if router_logits else None
        return cls(**kw)


def _positions_from_segments(segment_ids: torch.Tensor) -> torch.Tensor:
    """Positions restart at 0 at every segment boundary of a packed row."""
    B, T = segment_ids.shape
    idx = torch.arange(T, device=segment_ids.device)[None].expand(B, T)
    change = torch.ones_like(segment_ids, dtype=torch.bool)
    change[:, 1:] = segment_ids[:, 1:] != segment_ids[:, :-1]
    start = torch.where(change, idx, torch.zeros_like(idx)).cummax(dim=1).values
    return idx - start


class DecoderForCausalLM(EasyDeLBaseModule):
    """Backbone + LM head. ``apply_lm_head=False`` returns hidden states only (chunked loss, serving)."""

    backbone_cls: type[DecoderModel] = DecoderModel
    loss_type = "ForCausalLM"

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.model = type(self).backbone_cls(config, dtype, param_dtype, precision, rngs)
        spec = self.model.spec
        self.spec = spec
        if not spec.tie_embeddings:
            tp_size, tp_rank, tp_group = 1, 0, None  # vocab-parallel head is set up by parallel.tp when enabled
            self.lm_head = ColumnParallelLinear(spec.hidden_size, spec.vocab_size, bias=spec.lm_head_bias,
                                                dtype=self.param_dtype, init_std=spec.init_std)
        else:
            self.lm_head = None

    def can_generate(self) -> bool:
        return True

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def lm_head_weight(self) -> torch.Tensor:
        return self.model.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    def lm_head_bias(self):
        return None if self.lm_head is None else self.lm_head.bias

    def apply_lm_head(self, hidden: torch.Tensor) -> torch.Tensor:
        spec = self.spec
        logits = F.linear(hidden, self.lm_head_weight(), self.lm_head_bias())
        if spec.logit_scale is not None:
            logits = logits * spec.logit_scale
        if spec.logit_softcap:
            logits = torch.tanh(logits.float() / spec.logit_softcap).mul_(spec.logit_softcap).to(logits.dtype)
        return logits

    def apply_lm_head_vocab_parallel(self, hidden: torch.Tensor, group) -> torch.Tensor:
        """Serving under tensor parallelism: every rank multiplies by its slice of the (replicated) head's rows and
        the slices of the logits are gathered, so a decode step streams ``vocab / tp`` rows of the head per GPU
        instead of all of them. Same values as :meth:`apply_lm_head` (each logit is one dot product either way)."""
        import torch.distributed as dist

        n, r = dist.get_world_size(group), dist.get_rank(group)
        W = self.lm_head_weight()
        V = W.shape[0]
        if n == 1 or V % (8 * n) or hidden.dim() != 2 or torch.is_grad_enabled():
            return self.apply_lm_head(hidden)
        vs = V // n
        bias = self.lm_head_bias()
        part = F.linear(hidden, W[r * vs:(r + 1) * vs], None if bias is None else bias[r * vs:(r + 1) * vs])
        full = torch.empty(n * hidden.shape[0], vs, dtype=part.dtype, device=part.device)
        dist.all_gather_into_tensor(full, part.contiguous(), group=group)
        logits = full.view(n, hidden.shape[0], vs).permute(1, 0, 2).reshape(hidden.shape[0], V)
        spec = self.spec
        if spec.logit_scale is not None:
            logits = logits * spec.logit_scale
        if spec.logit_softcap:
            logits = torch.tanh(logits.float() / spec.logit_softcap).mul_(spec.logit_softcap).to(logits.dtype)
        return logits

    def make_lm_head_fn(self):
        return self.apply_lm_head

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, segment_ids=None, inputs_embeds=None,
                past_key_values=None, cache_metadata=None, output_hidden_states=False, output_router_logits=False,
                apply_lm_head: bool = True, labels: torch.Tensor | None = None, sequence_parallel: bool = False,
                **kw):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         segment_ids=segment_ids, inputs_embeds=inputs_embeds, past_key_values=past_key_values,
                         cache_metadata=cache_metadata, output_hidden_states=output_hidden_states,
                         output_router_logits=output_router_logits, deepstack_embeds=kw.get("deepstack_embeds"),
                         sequence_parallel=sequence_parallel and not apply_lm_head)
        hidden = out.last_hidden_state
        logits = self.apply_lm_head(hidden) if apply_lm_head else None
        rl = getattr(out, "router_logits", None)
        if self.spec.moe is not None:
            aux = None
            if rl and self.spec.moe.aux_loss_coef:
                aux = auxiliary_load_balancing_loss_func(rl, self.spec.moe.num_experts, self.spec.moe.top_k,
                                                         attention_mask)
            return MoeCausalLMOutput(logits=logits, last_hidden_state=hidden, hidden_states=out.hidden_states,
                                     past_key_values=out.past_key_values, router_logits=rl, aux_loss=aux)
        return CausalLMOutput(logits=logits, last_hidden_state=hidden, hidden_states=out.hidden_states,
                              past_key_values=out.past_key_values)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        call = dict(call)
        call["apply_lm_head"] = False
        if getattr(self.model, "sp_capable", False) and type(self).forward is DecoderForCausalLM.forward:
            call["sequence_parallel"] = True   # tensor-parallel dense stacks keep the token rows sharded
        cp_group = getattr(self.model, "cp_group", None)
        if cp_group is not None:
            import torch.distributed as dist

            from ...parallel import context_parallel as CP

            if not call.pop("labels_shifted", False):
                # the whole sequence came in: keep this rank's slice (labels shifted before the cut)
                keys = set(call) | {"position_ids"}
                b = CP.shard_batch({**call, "labels": labels}, dist.get_rank(cp_group), dist.get_world_size(cp_group),
                                   self.model.cp_layout)
                labels = b["labels"]
                call = {k: v for k, v in b.items() if k in keys}
            call.pop("attention_mask", None)        # folded into the labels; the layers see every token
        else:
            call.pop("labels_shifted", None)
        attention_mask = call.get("attention_mask")
        out = self(**call)
        if attention_mask is not None:
            labels = torch.where(attention_mask.bool(), labels, torch.full_like(labels, loss_config.ignore_index))
        spec = self.spec
        hidden = out.last_hidden_state
        if spec.logit_scale is not None:
            hidden = hidden * spec.logit_scale
        if cp_group is not None:
            # Sequence sharded over the ``sp`` axis: this rank computes the loss terms of its own tokens, normalised
            # by the group-wide token count; the loss is the sum over the group and EVERY parameter's gradient is a
            # partial sum (``cp_partial_grads``, summed over the group before the update).
            from ...parallel import tp as tpar

            metrics = causal_lm_loss_from_hidden(hidden, self.lm_head_weight(), labels, loss_config,
                                                 lm_head_bias=self.lm_head_bias(), softcap=spec.logit_softcap,
                                                 chunk_size=getattr(self.config, "lmhead_chunksize", None),
                                                 loss_scale=loss_scale, already_shifted=True, count_group=cp_group,
                                                 **loss_kwargs)
            metrics.loss = tpar.sum_value_over_group(metrics.loss, cp_group)
            if torch.is_grad_enabled():
                self.cp_partial_grads = True
            return out, metrics
        sp = getattr(self.model, "sp", None)
        if sp is not None and sp.active:
            # Every rank holds the hidden states of its own rows: it computes the loss terms of those rows
            # (normalised by the group-wide token count), so the loss is the sum over the group and every
            # replicated parameter's gradient is a partial sum (``sp_partial_grads``, summed before the update).
            from ...parallel import tp as tpar

            shifted = labels
            if loss_config.shift_tokens:
                shifted = torch.full_like(labels, loss_config.ignore_index)
                shifted[..., :-1] = labels[..., 1:]
            metrics = causal_lm_loss_from_hidden(hidden, self.lm_head_weight(), tpar.shard_rows(sp, shifted),
                                                 loss_config, lm_head_bias=self.lm_head_bias(),
                                                 softcap=spec.logit_softcap,
                                                 chunk_size=getattr(self.config, "lmhead_chunksize", None),
                                                 loss_scale=loss_scale, already_shifted=True, count_group=sp.group,
                                                 **loss_kwargs)
            metrics.loss = tpar.sum_value_over_group(metrics.loss, sp.group)
            if torch.is_grad_enabled():
                self.sp_partial_grads = True
            return out, metrics
        metrics = causal_lm_loss_from_hidden(hidden, self.lm_head_weight(), labels, loss_config,
                                             lm_head_bias=self.lm_head_bias(), softcap=spec.logit_softcap,
                                             chunk_size=getattr(self.config, "lmhead_chunksize", None),
                                             loss_scale=loss_scale, **loss_kwargs)
        aux = getattr(out, "aux_loss", None)
        if aux is not None and spec.moe is not None and spec.moe.aux_loss_coef:
            # the auxiliary loss is added to the training loss (easydel/infra/base_module.py:2791-2793)
            metrics.loss = metrics.loss + spec.moe.aux_loss_coef * aux * loss_scale
            metrics.other_metrics = {"aux_loss": aux.detach()}
        if spec.moe is not None and torch.is_grad_enabled():
            # per-block losses the blocks computed themselves (lbl_coef / rzl_coef carry their weights)
            extra: dict[str, torch.Tensor] = {}
            for layer in self.model.layers:
                for k, v in getattr(getattr(layer, "mlp", None), "last_aux_losses", {}).items():
                    extra[k] = extra[k] + v if k in extra else v
            if extra:
                metrics.loss = metrics.loss + sum(extra.values()) * loss_scale
                metrics.other_metrics = {**(metrics.other_metrics or {}), **{k: v.detach() for k, v in extra.items()}}
        return out, metrics


class DecoderForSequenceClassification(EasyDeLBaseModule):
    backbone_cls: type[DecoderModel] = DecoderModel
    loss_type = "ForSequenceClassification"

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.model = type(self).backbone_cls(config, dtype, param_dtype, precision, rngs)
        self.num_labels = getattr(config, "num_labels", 2)
        self.score = ColumnParallelLinear(self.model.spec.hidden_size, self.num_labels, bias=False,
                                          dtype=self.param_dtype, init_std=self.model.spec.init_std)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, segment_ids=None, inputs_embeds=None,
                labels=None, **kw):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         segment_ids=segment_ids, inputs_embeds=inputs_embeds)
        h = out.last_hidden_state
        B, T = h.shape[:2]
        if attention_mask is not None:
            last = (attention_mask.long() * torch.arange(T, device=h.device)[None]).argmax(-1)
        elif input_ids is not None and getattr(self.config, "pad_token_id", None) is not None:
            nonpad = (input_ids != self.config.pad_token_id).long()
            last = (nonpad * torch.arange(T, device=h.device)[None]).argmax(-1)
        else:
            last = torch.full((B,), T - 1, device=h.device, dtype=torch.long)
        pooled = h[torch.arange(B, device=h.device), last]
        logits = self.score(pooled)
        return SequenceClassifierOutput(logits=logits, hidden_states=out.hidden_states)

    def _compute_task_loss(self, labels, loss_config, loss_scale, call, loss_kwargs):
        out = self(**call)
        m = ForSequenceClassificationLoss(out.logits, labels, loss_config)
        m.loss = m.loss * loss_scale
        return out, m
