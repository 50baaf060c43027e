"""Llama-4 multimodal: the vision encoder, its pixel-shuffle adapter, the one-layer projector and the Llama-4 text
decoder (easydel/modules/llama4/modeling_llama4.py:1096-2371; the text decoder is the ``llama4_text`` family).

The encoder cuts a tile into patches with an unfold + one GEMM, appends the class token *after* the patches, adds a
learned position table and runs pre-LayerNorm blocks with bidirectional attention. Query and key pairs are rotated by
2-D angles: the first quarter of the head's frequencies turn with the patch column, the second quarter with the row
(both counted from 1), pairs interleaved; the class token is not rotated. After the final LayerNorm the class token
is dropped and the ``side x side`` grid is pixel-shuffled by ``pixel_shuffle_ratio`` (0.5: every 2 x 2 neighbourhood
becomes one row of four times the channels) and sent through a two-layer GELU MLP. ``multi_modal_projector`` maps the
result to the text width, and the rows overwrite the embeddings of the ``image_token_index`` placeholders.
"""

from __future__ import annotations

import torch
import torch.nn.functional as tF
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.modeling_outputs import BaseModelOutput
from ...layers.attention import Attention
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import PlainMLP
from ...layers.norms import LayerNorm
from ...layers.rotary import RotaryEmbedding
from .._base.vlm import VLMConfig, VLMForConditionalGeneration


@register_config("llama4_vision_model")
class Llama4VisionConfig(EasyDeLBaseConfig):
    model_type = "llama4_vision_model"
    use_class_token = True
    hf_config_keys = ("hidden_size", "hidden_act", "num_hidden_layers", "num_attention_heads", "num_channels",
                      "intermediate_size", "vision_output_dim", "image_size", "patch_size", "norm_eps",
                      "vision_feature_select_strategy", "pixel_shuffle_ratio", "projector_input_dim",
                      "projector_output_dim", "multi_modal_projector_bias", "rope_theta")

    def __init__(self, hidden_size=768, hidden_act="gelu", num_hidden_layers=34, num_attention_heads=16,
                 num_channels=3, intermediate_size=5632, vision_output_dim=7680, image_size=448, patch_size=14,
                 norm_eps=1e-5, vision_feature_select_strategy="default", initializer_range=0.02,
                 pixel_shuffle_ratio=0.5, projector_input_dim=4096, projector_output_dim=4096,
                 multi_modal_projector_bias=False, projector_dropout=0.0, attention_dropout=0.0, rope_theta=10000.0,
                 rope_parameters=None, **kw):
        self.hidden_size, self.hidden_act, self.num_hidden_layers = hidden_size, hidden_act, num_hidden_layers
        self.num_attention_heads, self.num_channels, self.intermediate_size = num_attention_heads, num_channels, \
            intermediate_size
        self.vision_output_dim, self.image_size, self.patch_size, self.norm_eps = vision_output_dim, image_size, \
            patch_size, norm_eps
        self.vision_feature_select_strategy, self.initializer_range = vision_feature_select_strategy, \
            initializer_range
        self.pixel_shuffle_ratio, self.projector_input_dim = pixel_shuffle_ratio, projector_input_dim
        self.projector_output_dim, self.multi_modal_projector_bias = projector_output_dim, multi_modal_projector_bias
        self.projector_dropout, self.attention_dropout = projector_dropout, attention_dropout
        if isinstance(rope_parameters, dict) and "rope_theta" in rope_parameters:
            rope_theta = rope_parameters["rope_theta"]
        self.rope_theta = rope_theta
        super().__init__(**kw)


def vision_rotary(head_dim: int, side: int, base: float) -> RotaryEmbedding:
    """Tables ``[side * side + 1, head_dim / 2]`` for patch ``row * side + col``; the last row (class token) is the
    identity rotation."""
    rot = RotaryEmbedding(head_dim, head_dim, 1, base, is_neox_style=False)
    fd = head_dim // 2
    freq = 1.0 / (base ** (torch.arange(0, fd, 2)[: fd // 2].float() / fd))
    idx = torch.arange(side * side)
    ang = torch.cat([torch.outer((idx % side + 1).float(), freq), torch.outer((idx // side + 1).float(), freq)], -1)
    ang = torch.cat([ang, torch.zeros(1, ang.shape[1])])
    rot.cos, rot.sin, rot.max_position = ang.cos(), ang.sin(), side * side + 1
    return rot


def pixel_shuffle(x: torch.Tensor, ratio: float) -> torch.Tensor:
    """``[B, side*side, C]`` -> ``[B, side*side*ratio^2, C / ratio^2]``: neighbouring grid cells are folded into the
    channel axis (width first, then height), as the adapter's weights expect."""
    B, n, C = x.shape
    side = int(round(n ** 0.5))
    x = x.view(B, side, int(side * ratio), int(C / ratio)).permute(0, 2, 1, 3)
    x = x.reshape(B, int(side * ratio), int(side * ratio), int(C / ratio ** 2)).permute(0, 2, 1, 3)
    return x.reshape(B, -1, x.shape[-1])


class Llama4UnfoldConvolution(nn.Module):
    """Patch embedding as unfold + GEMM (weight ``[hidden, channels * patch * patch]``, no bias)."""

    def __init__(self, c: Llama4VisionConfig, dtype):
        super().__init__()
        self.patch = c.patch_size
        self.linear = ColumnParallelLinear(c.num_channels * c.patch_size ** 2, c.hidden_size, bias=False, dtype=dtype,
                                           init_std=c.initializer_range)

    def forward(self, pixel_values):
        cols = tF.unfold(pixel_values.to(self.linear.weight.dtype), self.patch, stride=self.patch)
        return self.linear(cols.transpose(1, 2).contiguous())


class Llama4VisionEncoderLayer(nn.Module):
    def __init__(self, c: Llama4VisionConfig, idx: int, dtype, rotary):
        super().__init__()
        hd = c.hidden_size // c.num_attention_heads
        self.input_layernorm = LayerNorm(c.hidden_size, 1e-5, dtype=dtype)
        self.self_attn = Attention(c.hidden_size, c.num_attention_heads, c.num_attention_heads, hd, layer_idx=idx,
                                   bias=True, o_bias=True, rope=None, causal=False, dtype=dtype,
                                   init_std=c.initializer_range)
        self.self_attn.rotary = rotary
        self.post_attention_layernorm = LayerNorm(c.hidden_size, 1e-5, dtype=dtype)
        self.mlp = PlainMLP(c.hidden_size, c.intermediate_size, "gelu", True, dtype, c.initializer_range)

    def forward(self, x, pos):
        x = x + self.self_attn(self.input_layernorm(x), pos)
        return x + self.mlp(self.post_attention_layernorm(x))


class Llama4VisionEncoder(nn.Module):
    def __init__(self, c, dtype, rotary):
        super().__init__()
        self.layers = nn.ModuleList([Llama4VisionEncoderLayer(c, i, dtype, rotary)
                                     for i in range(c.num_hidden_layers)])


class Llama4VisionMLP2(nn.Module):
    """The adapter's MLP: GELU after *both* layers, no biases."""

    def __init__(self, c: Llama4VisionConfig, dtype):
        super().__init__()
        inner = int(c.hidden_size / c.pixel_shuffle_ratio ** 2)
        self.fc1 = ColumnParallelLinear(inner, c.projector_input_dim, bias=False, dtype=dtype,
                                        init_std=c.initializer_range)
        self.fc2 = ColumnParallelLinear(c.projector_output_dim, c.projector_output_dim, bias=False, dtype=dtype,
                                        init_std=c.initializer_range)

    def forward(self, x):
        return tF.gelu(self.fc2(tF.gelu(self.fc1(x))))


class Llama4VisionPixelShuffleMLP(nn.Module):
    def __init__(self, c, dtype):
        super().__init__()
        self.ratio = c.pixel_shuffle_ratio
        self.mlp = Llama4VisionMLP2(c, dtype)

    def forward(self, x):
        return self.mlp(pixel_shuffle(x, self.ratio).contiguous())


class Llama4VisionTransformer(nn.Module):
    """Parameter names as in the checkpoints' ``vision_model.*`` subtree."""

    def __init__(self, c: Llama4VisionConfig, dtype):
        super().__init__()
        self.cfg = c
        self.side = c.image_size // c.patch_size
        n = self.side ** 2 + 1
        scale = c.hidden_size ** -0.5
        self.patch_embedding = Llama4UnfoldConvolution(c, dtype)
        self.class_embedding = nn.Parameter(scale * torch.randn(c.hidden_size, dtype=dtype))
        self.positional_embedding_vlm = nn.Parameter(scale * torch.randn(n, c.hidden_size, dtype=dtype))
        self.layernorm_pre = LayerNorm(c.hidden_size, 1e-5, dtype=dtype)
        self.layernorm_post = LayerNorm(c.hidden_size, 1e-5, dtype=dtype)
        rotary = vision_rotary(c.hidden_size // c.num_attention_heads, self.side, c.rope_theta)
        self.model = Llama4VisionEncoder(c, dtype, rotary)
        self.vision_adapter = Llama4VisionPixelShuffleMLP(c, dtype)

    def forward(self, pixel_values, output_hidden_states: bool = False):
        """``pixel_values`` ``[tiles, C, image_size, image_size]`` -> ``[tiles, side^2 * ratio^2, projector_output_dim]``."""
        x = self.patch_embedding(pixel_values)
        x = torch.cat([x, self.class_embedding.to(x.dtype).expand(x.shape[0], 1, -1)], 1)
        x = self.layernorm_pre(x + self.positional_embedding_vlm.to(x.dtype))
        B, T, _ = x.shape
        pos = torch.arange(T, device=x.device)[None].expand(B, T)
        hs = [x] if output_hidden_states else None
        for layer in self.model.layers:
            x = layer(x, pos)
            if hs is not None:
                hs.append(x)
        x = self.layernorm_post(x)[:, :-1]
        return BaseModelOutput(last_hidden_state=self.vision_adapter(x), hidden_states=tuple(hs) if hs else None)


@register_module(TaskType.BASE_VISION, config=Llama4VisionConfig, model_type="llama4_vision_model",
                 layernorm_names=["input_layernorm", "post_attention_layernorm", "layernorm_pre", "layernorm_post"])
class Llama4VisionModel(EasyDeLBaseModule):
    hf_keeps_fused = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.vision_model = Llama4VisionTransformer(config, self.param_dtype)

    def hf_rename_in(self, sd):
        # a stand-alone vision checkpoint has no ``vision_model.`` prefix
        return {("vision_model." + k if not k.startswith("vision_model.") else k): v for k, v in sd.items()}

    def hf_rename_out(self, sd):
        return {k[len("vision_model."):]: v for k, v in sd.items()}

    def forward(self, pixel_values, output_hidden_states=False, **_):
        return self.vision_model(pixel_values, output_hidden_states)


@register_config("llama4")
class Llama4Config(VLMConfig):
    model_type = "llama4"
    vision_default, text_default = "llama4_vision_model", "llama4_text"

    def __init__(self, vision_config=None, text_config=None, boi_token_index=200080, eoi_token_index=200081,
                 image_token_index=200092, **kw):
        kw = self._init_parts(vision_config, text_config, image_token_index, kw)
        self.boi_token_index, self.eoi_token_index = boi_token_index, eoi_token_index
        super().__init__(**kw)


class Llama4MultiModalProjector(nn.Module):
    def __init__(self, c: Llama4Config, dtype):
        super().__init__()
        self.linear_1 = ColumnParallelLinear(c.vision_config.vision_output_dim, c.text_config.hidden_size, bias=False,
                                             dtype=dtype, init_std=c.vision_config.initializer_range)

    def forward(self, x):
        return self.linear_1(x)


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Llama4Config, model_type="llama4")
class Llama4ForConditionalGeneration(VLMForConditionalGeneration):
    """Checkpoint layout: ``vision_model.*``, ``multi_modal_projector.linear_1.weight``, ``language_model.model.*``
    and ``language_model.lm_head.weight``."""

    ignored_prefixes = ()
    hf_keeps_fused = ("experts",)      # the checkpoints store each layer's experts as one stacked tensor

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.vision_model = Llama4VisionTransformer(config.vision_config, pd)
        self.multi_modal_projector = Llama4MultiModalProjector(config, pd)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)

    def hf_rename_in(self, sd):
        out = {k: v for k, v in sd.items() if not k.startswith("language_model.")}
        lm = {k[len("language_model."):]: v for k, v in sd.items() if k.startswith("language_model.")}
        out.update({"language_model." + k: v for k, v in self.language_model.hf_rename_in(lm).items()})
        return out

    def hf_rename_out(self, sd):
        out = {k: v for k, v in sd.items() if not k.startswith("language_model.")}
        lm = {k[len("language_model."):]: v for k, v in sd.items() if k.startswith("language_model.")}
        out.update({"language_model." + k: v for k, v in self.language_model.hf_rename_out(lm).items()})
        return out

    def get_image_features(self, pixel_values: torch.Tensor, **_) -> torch.Tensor:
        feats = self.vision_model(pixel_values).last_hidden_state
        return self.multi_modal_projector(feats.reshape(-1, feats.shape[-1]))
