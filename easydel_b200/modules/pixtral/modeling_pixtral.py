"""Pixtral vision tower (easydel/modules/pixtral): RMSNorm blocks with gated MLPs, rotary positions on the 2-D
patch grid, images of different sizes packed into one sequence.

Every image is cut to ``(h // patch) x (w // patch)`` patches; the patches of all images of a call form one packed
sequence whose attention is block-diagonal per image (segment ids -> varlen attention, not causal). The rotary table
is indexed by ``row * max_side + col``: the first half of the frequencies turns with the row, the second half with
the column.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.modeling_outputs import BaseModelOutput
from ...layers.attention import Attention
from ...layers.mlp import GatedMLP
from ...layers.norms import RMSNorm
from ...layers.rotary import RotaryEmbedding
from .._base.families import _Renamer


@register_config("pixtral")
class PixtralVisionConfig(EasyDeLBaseConfig):
    model_type = "pixtral"
    use_class_token = False
    hf_config_keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_channels",
                      "image_size", "patch_size", "hidden_act", "head_dim", "rope_theta")

    def __init__(self, hidden_size=1024, intermediate_size=4096, num_hidden_layers=24, num_attention_heads=16,
                 num_channels=3, image_size=1024, patch_size=16, hidden_act="gelu", attention_dropout=0.0,
                 rope_theta=10000.0, head_dim=None, initializer_range=0.02, **kw):
        self.hidden_size, self.intermediate_size, self.num_hidden_layers = hidden_size, intermediate_size, \
            num_hidden_layers
        self.num_attention_heads, self.num_channels, self.image_size, self.patch_size = num_attention_heads, \
            num_channels, image_size, patch_size
        self.hidden_act, self.attention_dropout, self.rope_theta = hidden_act, attention_dropout, rope_theta
        self.head_dim = head_dim or hidden_size // num_attention_heads
        self.initializer_range = initializer_range
        super().__init__(**kw)


def grid_rotary(head_dim: int, side: int, base: float) -> RotaryEmbedding:
    """Rotary tables ``[side * side, head_dim / 2]`` for positions ``row * side + col``."""
    rot = RotaryEmbedding(head_dim, head_dim, 1, base, is_neox_style=True)
    freqs = 1.0 / (base ** (torch.arange(0, head_dim, 2).float() / head_dim))
    fh = torch.outer(torch.arange(side).float(), freqs[::2])
    fw = torch.outer(torch.arange(side).float(), freqs[1::2])
    ang = torch.cat([fh[:, None, :].expand(side, side, -1), fw[None, :, :].expand(side, side, -1)], -1)
    ang = ang.reshape(side * side, head_dim // 2)
    rot.cos, rot.sin, rot.max_position = ang.cos(), ang.sin(), side * side
    return rot


class PixtralLayer(nn.Module):
    def __init__(self, c: PixtralVisionConfig, idx: int, dtype, rotary):
        super().__init__()
        self.attention_norm = RMSNorm(c.hidden_size, 1e-5, dtype)
        self.attention = Attention(c.hidden_size, c.num_attention_heads, c.num_attention_heads, c.head_dim,
                                   layer_idx=idx, bias=False, o_bias=False, rope=None, causal=False, dtype=dtype,
                                   init_std=c.initializer_range)
        self.attention.rotary = rotary
        self.ffn_norm = RMSNorm(c.hidden_size, 1e-5, dtype)
        self.feed_forward = GatedMLP(c.hidden_size, c.intermediate_size, c.hidden_act, False, dtype,
                                     c.initializer_range)

    def forward(self, x, pos, seg):
        x = x + self.attention(self.attention_norm(x), pos, segment_ids=seg)
        return x + self.feed_forward(self.ffn_norm(x))


class PixtralTransformer(nn.Module):
    def __init__(self, c: PixtralVisionConfig, dtype):
        super().__init__()
        self.cfg = c
        self.patch_conv = nn.Conv2d(c.num_channels, c.hidden_size, c.patch_size, c.patch_size, bias=False, dtype=dtype)
        self.ln_pre = RMSNorm(c.hidden_size, 1e-5, dtype)
        self.side = c.image_size // c.patch_size
        rotary = grid_rotary(c.head_dim, self.side, c.rope_theta)
        self.layers = nn.ModuleList([PixtralLayer(c, i, dtype, rotary) for i in range(c.num_hidden_layers)])

    def forward(self, pixel_values, image_sizes=None, output_hidden_states: bool = False):
        """``pixel_values`` ``[N, 3, H, W]`` (padded to a common size); ``image_sizes`` ``[(h, w)]`` per image.
        Returns the packed patch sequence ``[1, sum(h_i w_i / patch^2), D]``."""
        c = self.cfg
        N, _, H, W = pixel_values.shape
        if image_sizes is None:
            image_sizes = [(H, W)] * N
        emb = self.patch_conv(pixel_values.to(self.patch_conv.weight.dtype))
        rows, pos, seg = [], [], []
        for i, (h, w) in enumerate(image_sizes):
            gh, gw = int(h) // c.patch_size, int(w) // c.patch_size
            rows.append(emb[i, :, :gh, :gw].flatten(1).t())
            r = torch.arange(gh, device=emb.device)[:, None].expand(gh, gw)
            q = torch.arange(gw, device=emb.device)[None, :].expand(gh, gw)
            pos.append((r * self.side + q).reshape(-1))
            seg.append(torch.full((gh * gw,), i + 1, dtype=torch.int32, device=emb.device))
        x = self.ln_pre(torch.cat(rows)[None].contiguous())
        pos, seg = torch.cat(pos)[None], torch.cat(seg)[None]
        if N == 1:
            seg = None
        hs = [x] if output_hidden_states else None
        for layer in self.layers:
            x = layer(x, pos, seg)
            if hs is not None:
                hs.append(x)
        return BaseModelOutput(last_hidden_state=x, hidden_states=tuple(hs) if hs else None)


_REN = _Renamer([("transformer.layers.", "vision_model.layers."), ("patch_conv.", "vision_model.patch_conv."),
                 ("ln_pre.", "vision_model.ln_pre.")])


@register_module(TaskType.BASE_VISION, config=PixtralVisionConfig, model_type="pixtral",
                 layernorm_names=["attention_norm", "ffn_norm", "ln_pre"])
class PixtralVisionModel(EasyDeLBaseModule):
    hf_keeps_fused = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.vision_model = PixtralTransformer(config, self.param_dtype)

    def hf_rename_in(self, sd):
        return _REN.to_internal(self, sd)

    def hf_rename_out(self, sd):
        return _REN.to_hf(self, sd)

    def forward(self, pixel_values, image_sizes=None, output_hidden_states=False, **_):
        return self.vision_model(pixel_values, image_sizes, output_hidden_states)
