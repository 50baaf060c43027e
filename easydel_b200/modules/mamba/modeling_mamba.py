"""Mamba-1 and Falcon-Mamba (easydel/modules/mamba, falcon_mamba): attention-free selective state-space models.

Block: RMSNorm -> in_proj -> (x, z); x -> causal depth-wise conv1d + SiLU -> x_proj -> (dt, B, C);
dt_proj -> selective scan with A = -exp(A_log), skip D, gate SiLU(z) -> out_proj, residual add. Falcon-Mamba
applies a weight-free RMS norm to dt, B and C. Parameter names follow the Hugging Face checkpoints
(``backbone.layers.N.mixer.*``), so state dicts load without renaming. The recurrences run in ``ops/ssm.py``
(CUDA scan kernels on the GPU). Generation keeps a per-layer conv window and SSM state (:class:`MambaCache`).
"""

from __future__ import annotations

import math

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.loss_utils import LossConfig, causal_lm_loss_from_hidden
from ...infra.modeling_outputs import BaseModelOutput, CausalLMOutput
from ...layers.embeddings import Embed
from ...layers.linears import ColumnParallelLinear
from ...layers.norms import RMSNorm
from ...ops import functional as F
from ...ops import ssm


@register_config("mamba")
class MambaConfig(EasyDeLBaseConfig):
    model_type = "mamba"
    hf_config_keys = ("vocab_size", "hidden_size", "state_size", "num_hidden_layers", "layer_norm_epsilon", "expand",
                      "conv_kernel", "use_bias", "use_conv_bias", "hidden_act", "initializer_range",
                      "residual_in_fp32", "time_step_rank", "time_step_scale", "time_step_min", "time_step_max",
                      "time_step_init_scheme", "time_step_floor", "rescale_prenorm_residual", "tie_word_embeddings",
                      "intermediate_size")

    def __init__(self, vocab_size=50280, hidden_size=768, state_size=16, num_hidden_layers=32,
                 layer_norm_epsilon=1e-5, pad_token_id=0, bos_token_id=0, eos_token_id=0, expand=2, conv_kernel=4,
                 use_bias=False, use_conv_bias=True, hidden_act="silu", initializer_range=0.1, residual_in_fp32=True,
                 time_step_rank="auto", time_step_scale=1.0, time_step_min=0.001, time_step_max=0.1,
                 time_step_init_scheme="random", time_step_floor=1e-4, rescale_prenorm_residual=False,
                 use_cache=True, tie_word_embeddings=True, mixer_rms_eps=1e-6, **kw):
        self.vocab_size, self.hidden_size, self.state_size = vocab_size, hidden_size, state_size
        self.num_hidden_layers, self.layer_norm_epsilon = num_hidden_layers, layer_norm_epsilon
        self.expand, self.conv_kernel = expand, conv_kernel
        self.intermediate_size = kw.pop("intermediate_size", None) or int(expand * hidden_size)
        self.use_bias, self.use_conv_bias, self.hidden_act = use_bias, use_conv_bias, hidden_act
        self.initializer_range, self.residual_in_fp32 = initializer_range, residual_in_fp32
        self.time_step_rank = math.ceil(hidden_size / 16) if time_step_rank == "auto" else time_step_rank
        self.time_step_scale, self.time_step_min, self.time_step_max = time_step_scale, time_step_min, time_step_max
        self.time_step_init_scheme, self.time_step_floor = time_step_init_scheme, time_step_floor
        self.rescale_prenorm_residual, self.use_cache, self.mixer_rms_eps = rescale_prenorm_residual, use_cache, \
            mixer_rms_eps
        super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                         tie_word_embeddings=tie_word_embeddings, **kw)


@register_config("falcon_mamba")
class FalconMambaConfig(MambaConfig):
    model_type = "falcon_mamba"

    def __init__(self, vocab_size=50280, hidden_size=768, tie_word_embeddings=False, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, tie_word_embeddings=tie_word_embeddings, **kw)


class MambaCache:
    """Per-layer conv window ``[B, W-1, C]`` and SSM state ``[B, C, N]`` (fp32) for incremental decoding."""

    def __init__(self, config: MambaConfig, batch_size: int, device, dtype=torch.bfloat16):
        C, N, W = config.intermediate_size, config.state_size, config.conv_kernel
        self.conv = [torch.zeros(batch_size, W - 1, C, dtype=dtype, device=device)
                     for _ in range(config.num_hidden_layers)]
        self.ssm = [torch.zeros(batch_size, C, N, dtype=torch.float32, device=device)
                    for _ in range(config.num_hidden_layers)]
        self.seen = 0

    def seq_len(self) -> int:
        return self.seen

    def advance(self, n: int) -> None:
        self.seen += n


def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


class MambaMixer(nn.Module):
    def __init__(self, config: MambaConfig, layer_idx: int, dtype, norm_bcdt: bool = False):
        super().__init__()
        H, C, N, R, W = config.hidden_size, config.intermediate_size, config.state_size, config.time_step_rank, \
            config.conv_kernel
        self.C, self.N, self.R, self.W, self.layer_idx = C, N, R, W, layer_idx
        self.norm_bcdt, self.rms_eps = norm_bcdt, config.mixer_rms_eps
        std = config.initializer_range
        self.in_proj = ColumnParallelLinear(H, 2 * C, bias=config.use_bias, dtype=dtype, init_std=std)
        self.conv1d = nn.Conv1d(C, C, W, groups=C, padding=W - 1, bias=config.use_conv_bias, dtype=dtype)
        self.x_proj = ColumnParallelLinear(C, R + 2 * N, bias=False, dtype=dtype, init_std=std)
        self.dt_proj = ColumnParallelLinear(R, C, bias=True, dtype=dtype, init_std=R ** -0.5 * config.time_step_scale)
        self.A_log = nn.Parameter(torch.log(torch.arange(1, N + 1, dtype=torch.float32))[None].repeat(C, 1))
        self.D = nn.Parameter(torch.ones(C, dtype=torch.float32))
        self.out_proj = ColumnParallelLinear(C, H, bias=config.use_bias, dtype=dtype, init_std=std)
        with torch.no_grad():   # inverse-softplus of time steps log-uniform in [min, max]
            dt = torch.exp(torch.rand(C) * (math.log(config.time_step_max) - math.log(config.time_step_min))
                           + math.log(config.time_step_min)).clamp_min(config.time_step_floor)
            if self.dt_proj.bias.device.type != "meta":
                self.dt_proj.bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(self.dt_proj.bias.dtype))

    def forward(self, h: torch.Tensor, cache: MambaCache | None = None) -> torch.Tensor:
        B, T, _ = h.shape
        xz = self.in_proj(h)
        x, z = xz[..., : self.C], xz[..., self.C:]
        cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=h.device)
        xf = x.reshape(B * T, self.C)
        conv_state = cache.conv[self.layer_idx] if cache is not None else None
        xc = ssm.ragged_conv1d(xf, self.conv1d.weight[:, 0, :], self.conv1d.bias, cu, "silu", conv_state)
        p = self.x_proj(xc)
        dt, Bm, Cm = p[..., : self.R], p[..., self.R: self.R + self.N], p[..., self.R + self.N:]
        if self.norm_bcdt:
            dt, Bm, Cm = _rms(dt, self.rms_eps), _rms(Bm, self.rms_eps), _rms(Cm, self.rms_eps)
        delta = F.linear(dt, self.dt_proj.weight)          # bias is added inside the scan, before softplus
        A = -torch.exp(self.A_log.float())
        y = ssm.selective_scan(xc, delta.contiguous(), A, Bm.contiguous(), Cm.contiguous(), self.D,
                               z.reshape(B * T, self.C).contiguous(), self.dt_proj.bias.float(), True, cu,
                               cache.ssm[self.layer_idx] if cache is not None else None)
        return self.out_proj(y.view(B, T, self.C))


class MambaBlock(nn.Module):
    def __init__(self, config, layer_idx, dtype, norm_bcdt=False):
        super().__init__()
        self.norm = RMSNorm(config.hidden_size, config.layer_norm_epsilon, dtype)
        self.mixer = MambaMixer(config, layer_idx, dtype, norm_bcdt)

    def forward(self, x, cache=None):
        return x + self.mixer(self.norm(x), cache)


class _Backbone(nn.Module):
    def __init__(self, config, dtype, norm_bcdt):
        super().__init__()
        self.embeddings = Embed(config.vocab_size, config.hidden_size, dtype, config.initializer_range)
        self.layers = nn.ModuleList([MambaBlock(config, i, dtype, norm_bcdt) for i in range(config.num_hidden_layers)])
        self.norm_f = RMSNorm(config.hidden_size, config.layer_norm_epsilon, dtype)


@register_module(TaskType.BASE_MODULE, config=MambaConfig, model_type="mamba")
class MambaModel(EasyDeLBaseModule):
    norm_bcdt = False

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.backbone = _Backbone(config, self.param_dtype, type(self).norm_bcdt)

    def get_input_embeddings(self):
        return self.backbone.embeddings

    def init_cache(self, batch_size: int, max_length: int | None = None, **_):
        return MambaCache(self.config, batch_size, self.device, self.dtype)

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values=None, attention_mask=None,
                output_hidden_states=False, **_):
        x = self.backbone.embeddings(input_ids) if inputs_embeds is None else inputs_embeds
        if attention_mask is not None and x.shape[1] > 1:
            x = x * attention_mask[..., None].to(x.dtype)
        hs = [] if output_hidden_states else None
        for layer in self.backbone.layers:
            if hs is not None:
                hs.append(x)
            x = layer(x, past_key_values)
        x = self.backbone.norm_f(x)
        if hs is not None:
            hs.append(x)
        return BaseModelOutput(last_hidden_state=x, hidden_states=tuple(hs) if hs else None,
                               past_key_values=past_key_values)


@register_module(TaskType.CAUSAL_LM, config=MambaConfig, model_type="mamba")
class MambaForCausalLM(EasyDeLBaseModule):
    backbone_cls = MambaModel
    loss_type = "ForCausalLM"

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        inner = type(self).backbone_cls(config, dtype, param_dtype, precision, rngs)
        self.backbone = inner.backbone
        self._inner = [inner]     # not a submodule: its parameters are reachable through ``self.backbone``
        self.lm_head = None if config.tie_word_embeddings else ColumnParallelLinear(
            config.hidden_size, config.vocab_size, bias=False, dtype=self.param_dtype,
            init_std=config.initializer_range)

    def can_generate(self):
        return True

    def get_input_embeddings(self):
        return self.backbone.embeddings

    def lm_head_weight(self):
        return self.backbone.embeddings.weight if self.lm_head is None else self.lm_head.weight

    def lm_head_bias(self):
        return None

    def init_cache(self, batch_size: int, max_length: int | None = None, **_):
        return MambaCache(self.config, batch_size, self.device, self.dtype)

    def apply_lm_head(self, hidden):
        return F.linear(hidden, self.lm_head_weight())

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values=None, attention_mask=None,
                apply_lm_head: bool = True, output_hidden_states=False, **_):
        out = self._inner[0].forward(input_ids=input_ids, inputs_embeds=inputs_embeds, past_key_values=past_key_values,
                                     attention_mask=attention_mask, output_hidden_states=output_hidden_states)
        h = out.last_hidden_state
        return CausalLMOutput(logits=self.apply_lm_head(h) if apply_lm_head else None, last_hidden_state=h,
                              hidden_states=out.hidden_states, past_key_values=past_key_values)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        call = dict(call)
        call["apply_lm_head"] = False
        out = self(**call)
        am = call.get("attention_mask")
        if am is not None:
            labels = torch.where(am.bool(), labels, torch.full_like(labels, loss_config.ignore_index))
        m = causal_lm_loss_from_hidden(out.last_hidden_state, self.lm_head_weight(), labels, loss_config,
                                       loss_scale=loss_scale, **loss_kwargs)
        return out, m


@register_module(TaskType.BASE_MODULE, config=FalconMambaConfig, model_type="falcon_mamba")
class FalconMambaModel(MambaModel):
    norm_bcdt = True


@register_module(TaskType.CAUSAL_LM, config=FalconMambaConfig, model_type="falcon_mamba")
class FalconMambaForCausalLM(MambaForCausalLM):
    backbone_cls = FalconMambaModel


# ==================================================================================================== Mamba-2
@register_config("mamba2")
class Mamba2Config(EasyDeLBaseConfig):
    model_type = "mamba2"
    hf_config_keys = ("num_heads", "head_dim", "vocab_size", "hidden_size", "state_size", "num_hidden_layers",
                      "layer_norm_epsilon", "expand", "conv_kernel", "n_groups", "use_bias", "use_conv_bias",
                      "hidden_act", "initializer_range", "residual_in_fp32", "time_step_rank", "time_step_min",
                      "time_step_max", "time_step_floor", "time_step_limit", "rms_norm", "chunk_size",
                      "tie_word_embeddings")

    def __init__(self, num_heads=128, head_dim=64, vocab_size=32768, hidden_size=4096, state_size=128,
                 num_hidden_layers=64, layer_norm_epsilon=1e-5, pad_token_id=1, bos_token_id=0, eos_token_id=2,
                 expand=2, conv_kernel=4, n_groups=8, use_bias=False, use_conv_bias=True, hidden_act="silu",
                 initializer_range=0.1, residual_in_fp32=True, time_step_rank="auto", time_step_min=0.001,
                 time_step_max=0.1, time_step_floor=1e-4, time_step_limit=(0.0, float("inf")), rms_norm=True,
                 chunk_size=256, use_cache=True, tie_word_embeddings=False, **kw):
        self.num_heads, self.head_dim, self.vocab_size, self.hidden_size = num_heads, head_dim, vocab_size, hidden_size
        self.state_size, self.num_hidden_layers, self.layer_norm_epsilon = state_size, num_hidden_layers, \
            layer_norm_epsilon
        self.expand, self.conv_kernel, self.n_groups = expand, conv_kernel, n_groups
        self.intermediate_size = int(expand * hidden_size)
        if self.intermediate_size != num_heads * head_dim:
            raise ValueError(f"expand * hidden_size ({self.intermediate_size}) must equal num_heads * head_dim "
                             f"({num_heads * head_dim})")
        self.use_bias, self.use_conv_bias, self.hidden_act = use_bias, use_conv_bias, hidden_act
        self.initializer_range, self.residual_in_fp32 = initializer_range, residual_in_fp32
        self.time_step_rank = math.ceil(hidden_size / 16) if time_step_rank == "auto" else time_step_rank
        self.time_step_min, self.time_step_max, self.time_step_floor = time_step_min, time_step_max, time_step_floor
        self.time_step_limit, self.rms_norm, self.chunk_size, self.use_cache = tuple(time_step_limit), rms_norm, \
            chunk_size, use_cache
        super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                         tie_word_embeddings=tie_word_embeddings, **kw)


class Mamba2Cache:
    def __init__(self, config: Mamba2Config, batch_size: int, device, dtype=torch.bfloat16):
        conv_dim = config.intermediate_size + 2 * config.n_groups * config.state_size
        L = config.num_hidden_layers
        self.conv = [torch.zeros(batch_size, config.conv_kernel - 1, conv_dim, dtype=dtype, device=device)
                     for _ in range(L)]
        self.ssm = [torch.zeros(batch_size, config.num_heads, config.head_dim, config.state_size,
                                dtype=torch.float32, device=device) for _ in range(L)]
        self.seen = 0

    def seq_len(self):
        return self.seen

    def advance(self, n):
        self.seen += n


class Mamba2Mixer(nn.Module):
    def __init__(self, config: Mamba2Config, layer_idx: int, dtype):
        super().__init__()
        self.cfg, self.layer_idx = config, layer_idx
        H, I, G, N, NH = config.hidden_size, config.intermediate_size, config.n_groups, config.state_size, \
            config.num_heads
        self.conv_dim = I + 2 * G * N
        std = config.initializer_range
        self.in_proj = ColumnParallelLinear(H, I + self.conv_dim + NH, bias=config.use_bias, dtype=dtype, init_std=std)
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, config.conv_kernel, groups=self.conv_dim,
                                padding=config.conv_kernel - 1, bias=config.use_conv_bias, dtype=dtype)
        self.dt_bias = nn.Parameter(torch.zeros(NH, dtype=torch.float32))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, NH + 1, dtype=torch.float32)))
        self.D = nn.Parameter(torch.ones(NH, dtype=torch.float32))
        self.norm = _GatedRMSNorm(I, config.layer_norm_epsilon, dtype)
        self.out_proj = ColumnParallelLinear(I, H, bias=config.use_bias, dtype=dtype, init_std=std)
        with torch.no_grad():
            dt = torch.exp(torch.rand(NH) * (math.log(config.time_step_max) - math.log(config.time_step_min))
                           + math.log(config.time_step_min)).clamp_min(config.time_step_floor)
            if self.dt_bias.device.type != "meta":
                self.dt_bias.copy_(dt + torch.log(-torch.expm1(-dt)))

    def forward(self, h, cache: Mamba2Cache | None = None):
        c = self.cfg
        B, T, _ = h.shape
        I, G, N, NH, P = c.intermediate_size, c.n_groups, c.state_size, c.num_heads, c.head_dim
        proj = self.in_proj(h)
        gate, xbc, dt = proj[..., :I], proj[..., I:I + self.conv_dim], proj[..., I + self.conv_dim:]
        cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=h.device)
        xbc = ssm.ragged_conv1d(xbc.reshape(B * T, self.conv_dim), self.conv1d.weight[:, 0, :], self.conv1d.bias, cu,
                                "silu", cache.conv[self.layer_idx] if cache is not None else None)
        x, Bm, Cm = xbc[:, :I], xbc[:, I:I + G * N], xbc[:, I + G * N:]
        lo, hi = c.time_step_limit
        dtf = dt.reshape(B * T, NH)
        if lo > 0.0 or hi != float("inf"):      # clamp after softplus: done here, the scan then takes dt as given
            dtf = torch.nn.functional.softplus(dtf.float() + self.dt_bias).clamp(lo, hi).to(x.dtype)
            bias, sp = None, False
        else:
            bias, sp = self.dt_bias, True
        y = ssm.ssd_scan(x.reshape(B * T, NH, P).contiguous(), dtf.contiguous(), -torch.exp(self.A_log.float()),
                         Bm.reshape(B * T, G, N).contiguous(), Cm.reshape(B * T, G, N).contiguous(), self.D, bias, sp,
                         cu, cache.ssm[self.layer_idx] if cache is not None else None)
        y = self.norm(y.reshape(B, T, I), gate)
        return self.out_proj(y)


class _GatedRMSNorm(nn.Module):
    def __init__(self, dim, eps, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.eps = eps

    def forward(self, x, gate):
        xf = x.float() * torch.nn.functional.silu(gate.float())
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (self.weight.float() * xf).to(x.dtype)


class Mamba2Block(nn.Module):
    def __init__(self, config, layer_idx, dtype):
        super().__init__()
        self.norm = RMSNorm(config.hidden_size, config.layer_norm_epsilon, dtype)
        self.mixer = Mamba2Mixer(config, layer_idx, dtype)

    def forward(self, x, cache=None):
        return x + self.mixer(self.norm(x), cache)


class _Backbone2(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        self.embeddings = Embed(config.vocab_size, config.hidden_size, dtype, config.initializer_range)
        self.layers = nn.ModuleList([Mamba2Block(config, i, dtype) for i in range(config.num_hidden_layers)])
        self.norm_f = RMSNorm(config.hidden_size, config.layer_norm_epsilon, dtype)


@register_module(TaskType.BASE_MODULE, config=Mamba2Config, model_type="mamba2")
class Mamba2Model(MambaModel):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        EasyDeLBaseModule.__init__(self, config, dtype, param_dtype, precision, rngs)
        self.backbone = _Backbone2(config, self.param_dtype)

    def init_cache(self, batch_size: int, max_length: int | None = None, **_):
        return Mamba2Cache(self.config, batch_size, self.device, self.dtype)


@register_module(TaskType.CAUSAL_LM, config=Mamba2Config, model_type="mamba2")
class Mamba2ForCausalLM(MambaForCausalLM):
    backbone_cls = Mamba2Model

    def init_cache(self, batch_size: int, max_length: int | None = None, **_):
        return Mamba2Cache(self.config, batch_size, self.device, self.dtype)
