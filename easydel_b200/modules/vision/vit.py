"""Vision transformers used as image towers: CLIP-ViT and SigLIP-ViT (easydel/modules/clip, siglip).

Patch embedding (one strided convolution) + learned positions (+ class token and a pre-LayerNorm for CLIP), then
pre-LayerNorm encoder layers with bidirectional attention (the flash kernel with ``causal=False``) and a plain GELU
MLP, then a final LayerNorm. Parameter names follow the Hugging Face checkpoints under ``vision_model.*`` with two
substitutions (fused ``qkv_proj`` and ``o_proj``) handled by the renaming table.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.modeling_outputs import BaseModelOutput
from ...layers.attention import Attention
from ...layers.mlp import PlainMLP
from ...layers.norms import LayerNorm
from .._base.families import _Renamer


class _VisionConfigBase(EasyDeLBaseConfig):
    use_class_token = True
    hf_config_keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_channels",
                      "image_size", "patch_size", "hidden_act", "layer_norm_eps")

    def __init__(self, hidden_size=768, intermediate_size=3072, num_hidden_layers=12, num_attention_heads=12,
                 num_channels=3, image_size=224, patch_size=32, hidden_act="quick_gelu", layer_norm_eps=1e-5,
                 initializer_range=0.02, **kw):
        self.hidden_size, self.intermediate_size, self.num_hidden_layers = hidden_size, intermediate_size, \
            num_hidden_layers
        self.num_attention_heads, self.num_channels, self.image_size, self.patch_size = num_attention_heads, \
            num_channels, image_size, patch_size
        self.hidden_act, self.layer_norm_eps, self.initializer_range = hidden_act, layer_norm_eps, initializer_range
        super().__init__(**kw)


@register_config("clip_vision_model")
class CLIPVisionConfig(_VisionConfigBase):
    model_type = "clip_vision_model"
    use_class_token = True

    def __init__(self, **kw):   # an explicit constructor: the config base class generates one for classes without
        super().__init__(**kw)


@register_config("siglip_vision_model")
class SiglipVisionConfig(_VisionConfigBase):
    model_type = "siglip_vision_model"
    use_class_token = False

    def __init__(self, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6, patch_size=16, **kw):
        super().__init__(hidden_act=hidden_act, layer_norm_eps=layer_norm_eps, patch_size=patch_size, **kw)


class _EncoderLayer(nn.Module):
    def __init__(self, c, idx, dtype, causal: bool = False):
        super().__init__()
        hd = c.hidden_size // c.num_attention_heads
        self.layer_norm1 = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)
        self.self_attn = Attention(c.hidden_size, c.num_attention_heads, c.num_attention_heads, hd, layer_idx=idx,
                                   bias=True, o_bias=True, rope=None, causal=causal, dtype=dtype,
                                   init_std=c.initializer_range)
        self.layer_norm2 = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)
        self.mlp = PlainMLP(c.hidden_size, c.intermediate_size, c.hidden_act, True, dtype, c.initializer_range)

    def forward(self, x, pos, segment_ids=None):
        x = x + self.self_attn(self.layer_norm1(x), pos, segment_ids=segment_ids)
        return x + self.mlp(self.layer_norm2(x))


class VisionTransformer(nn.Module):
    def __init__(self, c, dtype):
        super().__init__()
        self.cfg = c
        n_patches = (c.image_size // c.patch_size) ** 2
        self.patch_embedding = nn.Conv2d(c.num_channels, c.hidden_size, c.patch_size, c.patch_size,
                                         bias=not c.use_class_token, dtype=dtype)
        if c.use_class_token:
            self.class_embedding = nn.Parameter(torch.randn(c.hidden_size, dtype=dtype) * c.initializer_range)
            self.pre_layrnorm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)
        self.position_embedding = nn.Embedding(n_patches + int(c.use_class_token), c.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([_EncoderLayer(c, i, dtype) for i in range(c.num_hidden_layers)])
        self.post_layernorm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)

    def forward(self, pixel_values: torch.Tensor, output_hidden_states: bool = False):
        c = self.cfg
        x = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        if c.use_class_token:
            x = torch.cat([self.class_embedding.expand(x.shape[0], 1, -1), x], 1)
        B, T, _ = x.shape
        pos = torch.arange(T, device=x.device)[None].expand(B, T)
        x = x + self.position_embedding(pos)
        if c.use_class_token:
            x = self.pre_layrnorm(x)
        hs = [x] if output_hidden_states else None
        for layer in self.layers:
            x = layer(x, pos)
            if hs is not None:
                hs.append(x)
        return BaseModelOutput(last_hidden_state=self.post_layernorm(x), hidden_states=tuple(hs) if hs else None)


VISION_RULES = [(".encoder.layers.", ".layers."), (".embeddings.class_embedding", ".class_embedding"),
                (".embeddings.patch_embedding.", ".patch_embedding."),
                (".embeddings.position_embedding.", ".position_embedding."), (".self_attn.out_proj.", ".self_attn.o_proj.")]
_REN = _Renamer(VISION_RULES)


class _VisionModelBase(EasyDeLBaseModule):
    hf_keeps_fused = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.vision_model = VisionTransformer(config, self.param_dtype)

    def hf_rename_in(self, sd):
        return _REN.to_internal(self, {k: v for k, v in sd.items() if not k.endswith("position_ids")})

    def hf_rename_out(self, sd):
        return _REN.to_hf(self, sd)

    def forward(self, pixel_values, output_hidden_states=False, **_):
        return self.vision_model(pixel_values, output_hidden_states)


@register_module(TaskType.BASE_VISION, config=CLIPVisionConfig, model_type="clip_vision_model",
                 layernorm_names=["layer_norm1", "layer_norm2", "pre_layrnorm", "post_layernorm"])
class CLIPVisionModel(_VisionModelBase):
    pass


@register_module(TaskType.BASE_VISION, config=SiglipVisionConfig, model_type="siglip_vision_model",
                 layernorm_names=["layer_norm1", "layer_norm2", "post_layernorm"])
class SiglipVisionModel(_VisionModelBase):
    pass
