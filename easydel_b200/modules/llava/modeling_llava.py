"""LLaVA: a vision tower, a two-layer projector and a Llama-family language model (easydel/modules/llava).

Image features are taken from one hidden layer of the tower (``vision_feature_layer``, default the one before
last; the class token is dropped under the ``default`` strategy), projected to the text width and written over
the embeddings of the ``image_token_index`` placeholders.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.factory import TaskType, register_config, register_module
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import ACT2FN
from .._base.vlm import VisionTower, VLMConfig, VLMForConditionalGeneration


@register_config("llava")
class LlavaConfig(VLMConfig):
    model_type = "llava"

    def __init__(self, vision_config=None, text_config=None, image_token_index=32000, projector_hidden_act="gelu",
                 vision_feature_select_strategy="default", vision_feature_layer=-2, image_seq_length=576,
                 multimodal_projector_bias=True, **kw):
        kw = self._init_parts(vision_config, text_config, image_token_index, kw)
        self.projector_hidden_act = projector_hidden_act
        self.vision_feature_select_strategy, self.vision_feature_layer = vision_feature_select_strategy, \
            vision_feature_layer
        self.image_seq_length, self.multimodal_projector_bias = image_seq_length, multimodal_projector_bias
        super().__init__(**kw)


class _Projector(nn.Module):
    def __init__(self, vis, txt, act, bias, dtype):
        super().__init__()
        self.linear_1 = ColumnParallelLinear(vis, txt, bias=bias, dtype=dtype)
        self.linear_2 = ColumnParallelLinear(txt, txt, bias=bias, dtype=dtype)
        self.act = act

    def forward(self, x):
        return self.linear_2(ACT2FN[self.act](self.linear_1(x)))


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=LlavaConfig, model_type="llava")
class LlavaForConditionalGeneration(VLMForConditionalGeneration):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.vision_tower = VisionTower(config.vision_config, pd)
        self.multi_modal_projector = _Projector(config.vision_config.hidden_size, config.text_config.hidden_size,
                                                config.projector_hidden_act, config.multimodal_projector_bias, pd)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)

    def get_image_features(self, pixel_values: torch.Tensor, **_) -> torch.Tensor:
        c = self.config
        out = self.vision_tower.vision_model(pixel_values, output_hidden_states=True)
        feats = out.hidden_states[c.vision_feature_layer]
        if c.vision_feature_select_strategy == "default" and c.vision_config.use_class_token:
            feats = feats[:, 1:]
        return self.multi_modal_projector(feats)
