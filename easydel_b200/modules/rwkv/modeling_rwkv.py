"""RWKV-4 (easydel/modules/rwkv): an attention-free recurrent language model.

Every block has a *time mixing* part (token shift, then the WKV recurrence: a per-channel exponentially decaying
average of past values weighted by ``exp(key)``, with a bonus ``time_first`` for the current token, gated by a sigmoid
receptance) and a *channel mixing* part (token shift, squared-ReLU key, sigmoid receptance gate). The WKV recurrence
is the CUDA kernel / oracle pair of ``ops/ssm.py``. Decoding carries, per layer, the previous token's two shifted
inputs and the three WKV accumulators.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.loss_utils import LossConfig, LossMetrics
from ...infra.modeling_outputs import BaseModelOutput, CausalLMOutput
from ...layers.linears import ColumnParallelLinear
from ...layers.norms import LayerNorm
from ...ops import functional as F
from ...ops import ssm


@register_config("rwkv")
class RwkvConfig(EasyDeLBaseConfig):
    model_type = "rwkv"
    attribute_map = {"max_position_embeddings": "context_length"}
    hf_config_keys = ("vocab_size", "context_length", "hidden_size", "num_hidden_layers", "attention_hidden_size",
                      "intermediate_size", "layer_norm_epsilon", "rescale_every")

    def __init__(self, vocab_size=50277, context_length=1024, hidden_size=4096, num_hidden_layers=32,
                 attention_hidden_size=None, intermediate_size=None, layer_norm_epsilon=1e-5, bos_token_id=0,
                 eos_token_id=0, rescale_every=6, tie_word_embeddings=False, initializer_range=0.02, **kw):
        self.vocab_size, self.context_length, self.hidden_size = vocab_size, context_length, hidden_size
        self.num_hidden_layers = num_hidden_layers
        self.attention_hidden_size = attention_hidden_size if attention_hidden_size is not None else hidden_size
        self.intermediate_size = intermediate_size if intermediate_size is not None else 4 * hidden_size
        self.layer_norm_epsilon, self.rescale_every = layer_norm_epsilon, rescale_every
        self.initializer_range = initializer_range
        super().__init__(bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                         tie_word_embeddings=tie_word_embeddings, **kw)


class RwkvState:
    """Per layer: previous input of time mixing, of channel mixing ``[B, H]``, and the WKV accumulators ``[B, 3, A]``."""

    def __init__(self, config: RwkvConfig, batch: int, device, dtype):
        L, H, A = config.num_hidden_layers, config.hidden_size, config.attention_hidden_size
        self.shift_att = torch.zeros(L, batch, H, dtype=dtype, device=device)
        self.shift_ffn = torch.zeros(L, batch, H, dtype=dtype, device=device)
        self.wkv = torch.zeros(L, batch, 3, A, dtype=torch.float32, device=device)
        self.wkv[:, :, 2] = -1e38
        self.seen = 0

    def seq_len(self):
        return self.seen

    def advance(self, n):
        self.seen += n


def _shift(x, prev):
    """Each token sees its predecessor; the first one sees ``prev`` (zeros at the start of a sequence)."""
    first = prev[:, None] if prev is not None else torch.zeros_like(x[:, :1])
    return torch.cat([first, x[:, :-1]], 1)


class RwkvSelfAttention(nn.Module):
    def __init__(self, c: RwkvConfig, idx: int, dtype):
        super().__init__()
        H, A = c.hidden_size, c.attention_hidden_size
        self.idx = idx
        self.time_decay = nn.Parameter(torch.zeros(A, dtype=dtype))
        self.time_first = nn.Parameter(torch.zeros(A, dtype=dtype))
        self.time_mix_key = nn.Parameter(torch.full((1, 1, H), 0.5, dtype=dtype))
        self.time_mix_value = nn.Parameter(torch.full((1, 1, H), 0.5, dtype=dtype))
        self.time_mix_receptance = nn.Parameter(torch.full((1, 1, H), 0.5, dtype=dtype))
        lin = lambda i, o: ColumnParallelLinear(i, o, bias=False, dtype=dtype, init_std=c.initializer_range)  # noqa: E731
        self.key, self.value, self.receptance, self.output = lin(H, A), lin(H, A), lin(H, A), lin(A, H)

    def forward(self, x, state: RwkvState | None):
        B, T, _ = x.shape
        sh = _shift(x, None if state is None else state.shift_att[self.idx])
        if state is not None:
            state.shift_att[self.idx] = x[:, -1]
        mix = lambda m: x * m + sh * (1 - m)  # noqa: E731
        k, v = self.key(mix(self.time_mix_key)), self.value(mix(self.time_mix_value))
        r = torch.sigmoid(self.receptance(mix(self.time_mix_receptance)))
        cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=x.device)
        A = k.shape[-1]
        wkv = ssm.wkv4(self.time_decay, self.time_first, k.reshape(B * T, A), v.reshape(B * T, A), cu,
                       None if state is None else state.wkv[self.idx])
        return self.output(r * wkv.view(B, T, A))


class RwkvFeedForward(nn.Module):
    def __init__(self, c: RwkvConfig, idx: int, dtype):
        super().__init__()
        H, I = c.hidden_size, c.intermediate_size
        self.idx = idx
        self.time_mix_key = nn.Parameter(torch.full((1, 1, H), 0.5, dtype=dtype))
        self.time_mix_receptance = nn.Parameter(torch.full((1, 1, H), 0.5, dtype=dtype))
        lin = lambda i, o: ColumnParallelLinear(i, o, bias=False, dtype=dtype, init_std=c.initializer_range)  # noqa: E731
        self.key, self.receptance, self.value = lin(H, I), lin(H, H), lin(I, H)

    def forward(self, x, state: RwkvState | None):
        sh = _shift(x, None if state is None else state.shift_ffn[self.idx])
        if state is not None:
            state.shift_ffn[self.idx] = x[:, -1]
        k = self.key(x * self.time_mix_key + sh * (1 - self.time_mix_key))
        r = torch.sigmoid(self.receptance(x * self.time_mix_receptance + sh * (1 - self.time_mix_receptance)))
        return r * self.value(torch.relu(k).square())


class RwkvBlock(nn.Module):
    def __init__(self, c: RwkvConfig, idx: int, dtype):
        super().__init__()
        if idx == 0:
            self.pre_ln = LayerNorm(c.hidden_size, c.layer_norm_epsilon, dtype=dtype)
        self.ln1 = LayerNorm(c.hidden_size, c.layer_norm_epsilon, dtype=dtype)
        self.ln2 = LayerNorm(c.hidden_size, c.layer_norm_epsilon, dtype=dtype)
        self.attention = RwkvSelfAttention(c, idx, dtype)
        self.feed_forward = RwkvFeedForward(c, idx, dtype)
        self.idx = idx

    def forward(self, x, state):
        if self.idx == 0:
            x = self.pre_ln(x)
        x = x + self.attention(self.ln1(x), state)
        return x + self.feed_forward(self.ln2(x), state)


class _Backbone(nn.Module):
    def __init__(self, c, dtype):
        super().__init__()
        self.embeddings = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dtype)
        self.blocks = nn.ModuleList([RwkvBlock(c, i, dtype) for i in range(c.num_hidden_layers)])
        self.ln_out = LayerNorm(c.hidden_size, c.layer_norm_epsilon, dtype=dtype)


@register_module(TaskType.BASE_MODULE, config=RwkvConfig, model_type="rwkv",
                 layernorm_names=["pre_ln", "ln1", "ln2", "ln_out"])
class RwkvModel(EasyDeLBaseModule):
    hf_keeps_fused = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.rwkv = _Backbone(config, self.param_dtype)

    def get_input_embeddings(self):
        return self.rwkv.embeddings

    def init_cache(self, batch_size: int, max_length: int | None = None, dtype=None, device=None):
        return RwkvState(self.config, batch_size, device or self.device, dtype or self.dtype)

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values: RwkvState | None = None,
                output_hidden_states=False, **_):
        x = self.rwkv.embeddings(input_ids) if inputs_embeds is None else inputs_embeds
        if x.dtype != self.dtype:
            x = x.to(self.dtype)
        hs = [] if output_hidden_states else None
        for blk in self.rwkv.blocks:
            if hs is not None:
                hs.append(x)
            x = blk(x, past_key_values)
        x = self.rwkv.ln_out(x)
        if hs is not None:
            hs.append(x)
        return BaseModelOutput(last_hidden_state=x, hidden_states=tuple(hs) if hs else None,
                               past_key_values=past_key_values)


@register_module(TaskType.CAUSAL_LM, config=RwkvConfig, model_type="rwkv",
                 layernorm_names=["pre_ln", "ln1", "ln2", "ln_out"])
class RwkvForCausalLM(EasyDeLBaseModule):
    loss_type = "ForCausalLM"
    hf_keeps_fused = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.rwkv = _Backbone(config, self.param_dtype)
        self.head = ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False, dtype=self.param_dtype)

    forward_backbone = RwkvModel.forward
    init_cache = RwkvModel.init_cache

    def can_generate(self):
        return True

    def get_input_embeddings(self):
        return self.rwkv.embeddings

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values=None, output_hidden_states=False,
                apply_lm_head: bool = True, **_):
        out = self.forward_backbone(input_ids=input_ids, inputs_embeds=inputs_embeds,
                                    past_key_values=past_key_values, output_hidden_states=output_hidden_states)
        logits = F.linear(out.last_hidden_state, self.head.weight) if apply_lm_head else None
        return CausalLMOutput(logits=logits, last_hidden_state=out.last_hidden_state,
                              hidden_states=out.hidden_states, past_key_values=past_key_values)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        out = self(input_ids=call.get("input_ids"), inputs_embeds=call.get("inputs_embeds"))
        lg = out.logits[:, :-1].float()
        loss = torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), labels[:, 1:].reshape(-1),
                                                 ignore_index=loss_config.ignore_index)
        return out, LossMetrics(loss=loss * loss_scale)
