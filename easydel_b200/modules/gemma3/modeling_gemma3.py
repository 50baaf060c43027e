"""Gemma-3 multimodal: SigLIP tower, average-pooling projector, Gemma-3 text model (easydel/modules/gemma3).

The tower's patch grid is average-pooled down to ``mm_tokens_per_image`` tokens, normalised with a (1 + w) RMSNorm
and multiplied by one projection matrix. The text model scales its token embeddings by sqrt(hidden) but takes the
image rows as they are, so the image rows are pre-divided by that factor before the merge. Attention over the merged
sequence is causal.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from ...infra.factory import TaskType, register_config, register_module
from ...layers.norms import RMSNorm
from .._base.vlm import VisionTower, VLMConfig, VLMForConditionalGeneration


@register_config("gemma3")
class Gemma3Config(VLMConfig):
    model_type = "gemma3"
    vision_default, text_default = "siglip_vision_model", "gemma3_text"

    def __init__(self, vision_config=None, text_config=None, mm_tokens_per_image=256, boi_token_index=255999,
                 eoi_token_index=256000, image_token_index=262144, initializer_range=0.02, **kw):
        kw.setdefault("tie_word_embeddings", True)
        kw = self._init_parts(vision_config, text_config, image_token_index, kw)
        self.mm_tokens_per_image, self.boi_token_index, self.eoi_token_index = mm_tokens_per_image, \
            boi_token_index, eoi_token_index
        self.initializer_range = initializer_range
        super().__init__(**kw)


class Gemma3MultiModalProjector(nn.Module):
    def __init__(self, c: Gemma3Config, dtype):
        super().__init__()
        v, t = c.vision_config, c.text_config
        self.mm_input_projection_weight = nn.Parameter(torch.randn(v.hidden_size, t.hidden_size, dtype=dtype) * 0.02)
        self.mm_soft_emb_norm = RMSNorm(v.hidden_size, v.layer_norm_eps, dtype, offset=1.0)
        self.side = v.image_size // v.patch_size
        self.kernel = self.side // int(math.isqrt(c.mm_tokens_per_image))

    def forward(self, feats):                       # [B, side*side, Dv]
        B, _, D = feats.shape
        x = feats.transpose(1, 2).reshape(B, D, self.side, self.side)
        x = torch.nn.functional.avg_pool2d(x, self.kernel, self.kernel).flatten(2).transpose(1, 2)
        x = self.mm_soft_emb_norm(x.contiguous())
        return torch.matmul(x, self.mm_input_projection_weight.to(x.dtype))


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Gemma3Config, model_type="gemma3")
class Gemma3ForConditionalGeneration(VLMForConditionalGeneration):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.vision_tower = VisionTower(config.vision_config, pd)
        self.multi_modal_projector = Gemma3MultiModalProjector(config, pd)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)

    def get_image_features(self, pixel_values, **_):
        feats = self.vision_tower.vision_model(pixel_values).last_hidden_state
        out = self.multi_modal_projector(feats)
        scale = self.language_model.spec.embed_scale
        return out / scale if scale else out
