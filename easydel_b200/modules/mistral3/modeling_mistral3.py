"""Mistral-3 (Mistral Small 3.x vision): Pixtral tower, learned 2x2 patch merger, two-layer projector, Mistral
language model (easydel/modules/mistral3).

The merger regroups every ``s x s`` neighbourhood of an image's patch grid (``s = spatial_merge_size``) into one row
of ``s*s*D`` channels and projects it back to ``D``; images keep their own sizes, so a call returns one packed
feature sequence that fills the image placeholders in order.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.factory import TaskType, register_config, register_module
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import ACT2FN
from ...layers.norms import RMSNorm
from .._base.families import _Renamer
from .._base.vlm import VLMConfig, VLMForConditionalGeneration
from ..pixtral.modeling_pixtral import PixtralTransformer


@register_config("mistral3")
class Mistral3Config(VLMConfig):
    model_type = "mistral3"
    vision_default, text_default = "pixtral", "mistral"

    def __init__(self, vision_config=None, text_config=None, image_token_index=10, projector_hidden_act="gelu",
                 vision_feature_layer=-1, multimodal_projector_bias=False, spatial_merge_size=2, **kw):
        kw = self._init_parts(vision_config, text_config, image_token_index, kw)
        self.projector_hidden_act, self.vision_feature_layer = projector_hidden_act, vision_feature_layer
        self.multimodal_projector_bias, self.spatial_merge_size = multimodal_projector_bias, spatial_merge_size
        super().__init__(**kw)


class Mistral3PatchMerger(nn.Module):
    def __init__(self, c: Mistral3Config, dtype):
        super().__init__()
        d = c.vision_config.hidden_size
        self.s, self.patch = c.spatial_merge_size, c.vision_config.patch_size
        self.merging_layer = ColumnParallelLinear(d * self.s ** 2, d, bias=False, dtype=dtype)

    def forward(self, feats, image_sizes):
        """feats ``[sum(h_i w_i), D]`` in image order -> ``[sum(h_i w_i / s^2), D]``."""
        s, d, out, o = self.s, feats.shape[-1], [], 0
        for h, w in image_sizes:
            gh, gw = int(h) // self.patch, int(w) // self.patch
            grid = feats[o:o + gh * gw].view(gh, gw, d)
            o += gh * gw
            # rows of the merged grid: channels ordered (d, dy, dx) as an unfold of the [d, gh, gw] image gives them
            g = grid.view(gh // s, s, gw // s, s, d).permute(0, 2, 4, 1, 3)
            out.append(g.reshape((gh // s) * (gw // s), d * s * s))
        return self.merging_layer(torch.cat(out))


class Mistral3MultiModalProjector(nn.Module):
    def __init__(self, c: Mistral3Config, dtype):
        super().__init__()
        v, t = c.vision_config.hidden_size, c.text_config.hidden_size
        self.norm = RMSNorm(v, c.text_config.rms_norm_eps, dtype)
        self.patch_merger = Mistral3PatchMerger(c, dtype)
        self.linear_1 = ColumnParallelLinear(v, t, bias=c.multimodal_projector_bias, dtype=dtype)
        self.linear_2 = ColumnParallelLinear(t, t, bias=c.multimodal_projector_bias, dtype=dtype)
        self.act = c.projector_hidden_act

    def forward(self, feats, image_sizes):
        x = self.patch_merger(self.norm(feats), image_sizes)
        return self.linear_2(ACT2FN[self.act](self.linear_1(x)))


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Mistral3Config, model_type="mistral3")
class Mistral3ForConditionalGeneration(VLMForConditionalGeneration):
    image_kwargs = ("image_sizes",)
    ignored_prefixes = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.vision_tower = PixtralTransformer(config.vision_config, pd)
        self.multi_modal_projector = Mistral3MultiModalProjector(config, pd)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)

    def _vision_renamer(self):
        return _Renamer([("vision_tower.transformer.layers.", "vision_tower.layers.")])

    def get_image_features(self, pixel_values, image_sizes=None, **_):
        if image_sizes is None:
            image_sizes = [tuple(pixel_values.shape[-2:])] * pixel_values.shape[0]
        image_sizes = [(int(h), int(w)) for h, w in (image_sizes.tolist() if isinstance(image_sizes, torch.Tensor)
                                                     else image_sizes)]
        out = self.vision_tower(pixel_values, image_sizes, output_hidden_states=True)
        feats = out.hidden_states[self.config.vision_feature_layer][0]
        return self.multi_modal_projector(feats, image_sizes)
