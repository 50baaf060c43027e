"""Aya Vision: SigLIP tower, pixel-shuffle + SwiGLU projector, Cohere-2 language model (easydel/modules/aya_vision).

Pixel shuffle folds each ``f x f`` neighbourhood of patches into the channel axis (``f = downsample_factor``), a
LayerNorm and a gated two-layer MLP then map ``Dv * f^2`` channels to the text width.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.factory import TaskType, register_config, register_module
from ...layers.linears import ColumnParallelLinear
from ...layers.norms import LayerNorm
from .._base.vlm import VisionTower, VLMConfig, VLMForConditionalGeneration


@register_config("aya_vision")
class AyaVisionConfig(VLMConfig):
    model_type = "aya_vision"
    vision_default, text_default = "siglip_vision_model", "cohere2"

    def __init__(self, vision_config=None, text_config=None, vision_feature_select_strategy="full",
                 vision_feature_layer=-1, downsample_factor=2, adapter_layer_norm_eps=1e-6, image_token_index=255036,
                 **kw):
        kw.setdefault("tie_word_embeddings", True)
        kw = self._init_parts(vision_config, text_config, image_token_index, kw)
        self.vision_feature_select_strategy, self.vision_feature_layer = vision_feature_select_strategy, \
            vision_feature_layer
        self.downsample_factor, self.adapter_layer_norm_eps = downsample_factor, adapter_layer_norm_eps
        super().__init__(**kw)


class AyaVisionMultiModalProjector(nn.Module):
    def __init__(self, c: AyaVisionConfig, dtype):
        super().__init__()
        self.f = c.downsample_factor
        d_in = c.vision_config.hidden_size * self.f ** 2
        align = getattr(c, "alignment_intermediate_size", None) or c.text_config.hidden_size
        self.layernorm = LayerNorm(d_in, c.adapter_layer_norm_eps, dtype=dtype)
        self.linear_1 = ColumnParallelLinear(d_in, align, bias=True, dtype=dtype)
        self.linear_2 = ColumnParallelLinear(align // 2, c.text_config.hidden_size, bias=True, dtype=dtype)

    def pixel_shuffle(self, x):                      # [B, S, D] with S a square
        B, S, D = x.shape
        h = w = int(S ** 0.5)
        f = self.f
        x = x.reshape(B, w, h, D)
        x = x.reshape(B, w, h // f, D * f).permute(0, 2, 1, 3)
        x = x.reshape(B, h // f, w // f, D * f * f).permute(0, 2, 1, 3)
        return x

    def forward(self, feats):
        x = self.linear_1(self.layernorm(self.pixel_shuffle(feats).contiguous()))
        a, g = x.chunk(2, dim=-1)
        return self.linear_2(torch.nn.functional.silu(g) * a)


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=AyaVisionConfig, model_type="aya_vision")
class AyaVisionForConditionalGeneration(VLMForConditionalGeneration):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.vision_tower = VisionTower(config.vision_config, pd)
        self.multi_modal_projector = AyaVisionMultiModalProjector(config, pd)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)
        # the multimodal head is a plain projection: Cohere's logit multiplier belongs to the text-only model
        self.language_model.spec.logit_scale = None

    def get_image_features(self, pixel_values, **_):
        c = self.config
        out = self.vision_tower.vision_model(pixel_values, output_hidden_states=True)
        feats = out.hidden_states[c.vision_feature_layer]      # encoder output before the tower's final LayerNorm
        return self.multi_modal_projector(feats)
