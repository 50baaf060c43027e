"""LLaVA: a vision tower, a two-layer projector and a Llama-family language model (easydel/modules/llava).

Image features are taken from one hidden layer of the tower (``vision_feature_layer``, default the one before
last; the class token is dropped under the ``default`` strategy), projected to the text width and written over
the embeddings of the ``image_token_index`` placeholders. Everything after that is the text model, so training,
generation and serving reuse the decoder path (``inputs_embeds``).
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module, registry
from ...infra.loss_utils import LossConfig
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import ACT2FN
from .._base.families import _Renamer
from ..vision.vit import VISION_RULES, VisionTransformer


@register_config("llava")
class LlavaConfig(EasyDeLBaseConfig):
    model_type = "llava"

    def __init__(self, vision_config=None, text_config=None, image_token_index=32000, projector_hidden_act="gelu",
                 vision_feature_select_strategy="default", vision_feature_layer=-2, image_seq_length=576,
                 multimodal_projector_bias=True, **kw):
        def build(c, default_type):
            if c is None:
                c = {}
            if isinstance(c, dict):
                c = dict(c)
                mt = c.pop("model_type", default_type)
                return registry.get_config(mt)(**c)
            return c

        self.vision_config = build(vision_config, "clip_vision_model")
        self.text_config = build(text_config, "llama")
        self.image_token_index, self.projector_hidden_act = image_token_index, projector_hidden_act
        self.vision_feature_select_strategy, self.vision_feature_layer = vision_feature_select_strategy, \
            vision_feature_layer
        self.image_seq_length, self.multimodal_projector_bias = image_seq_length, multimodal_projector_bias
        for k in ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads"):
            setattr(self, k, getattr(self.text_config, k, None))
        kw.setdefault("tie_word_embeddings", getattr(self.text_config, "tie_word_embeddings", False))
        super().__init__(**kw)

    def to_dict(self):
        d = super().to_dict()
        d["vision_config"] = self.vision_config.to_dict()
        d["text_config"] = self.text_config.to_dict()
        return d


class _Projector(nn.Module):
    def __init__(self, vis, txt, act, bias, dtype):
        super().__init__()
        self.linear_1 = ColumnParallelLinear(vis, txt, bias=bias, dtype=dtype)
        self.linear_2 = ColumnParallelLinear(txt, txt, bias=bias, dtype=dtype)
        self.act = act

    def forward(self, x):
        return self.linear_2(ACT2FN[self.act](self.linear_1(x)))


class _Tower(nn.Module):
    def __init__(self, cfg, dtype):
        super().__init__()
        self.vision_model = VisionTransformer(cfg, dtype)


_VISION = _Renamer(VISION_RULES)
_OUTER = _Renamer([("model.vision_tower.", "vision_tower."), ("model.multi_modal_projector.", "multi_modal_projector."),
                   ("model.language_model.", "language_model.model."), ("lm_head.", "language_model.lm_head.")])


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=LlavaConfig, model_type="llava")
class LlavaForConditionalGeneration(EasyDeLBaseModule):
    loss_type = "ForCausalLM"
    hf_keeps_fused = ()

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.vision_tower = _Tower(config.vision_config, pd)
        self.multi_modal_projector = _Projector(config.vision_config.hidden_size, config.text_config.hidden_size,
                                                config.projector_hidden_act, config.multimodal_projector_bias, pd)
        reg = registry.get_module_registration(TaskType.CAUSAL_LM, config.text_config.model_type)
        self.language_model = reg.module(config.text_config, dtype, param_dtype, precision, rngs)

    # weight-name maps: the language model keeps its own fused-projection handling
    def hf_rename_in(self, sd):
        sd = {k: v for k, v in sd.items() if not k.endswith("position_ids")}
        vis = {k: v for k, v in sd.items() if ".vision_tower." in k or k.startswith("vision_tower.")}
        rest = {k: v for k, v in sd.items() if k not in vis}
        out = _OUTER.to_internal(self, rest)
        out.update(_OUTER.to_internal(self, _VISION.to_internal(self, vis)))
        return out

    def hf_rename_out(self, sd):
        vis = {k: v for k, v in sd.items() if k.startswith("vision_tower.")}
        rest = {k: v for k, v in sd.items() if k not in vis}
        out = _OUTER.to_hf(self, rest)
        out.update(_OUTER.to_hf(self, _VISION.to_hf(self, vis)))
        return out

    @property
    def spec(self):
        return self.language_model.spec

    def can_generate(self):
        return True

    def get_input_embeddings(self):
        return self.language_model.get_input_embeddings()

    def lm_head_weight(self):
        return self.language_model.lm_head_weight()

    def lm_head_bias(self):
        return self.language_model.lm_head_bias()

    def apply_lm_head(self, h):
        return self.language_model.apply_lm_head(h)

    def init_cache(self, *a, **kw):
        return self.language_model.init_cache(*a, **kw)

    def get_image_features(self, pixel_values: torch.Tensor) -> torch.Tensor:
        c = self.config
        out = self.vision_tower.vision_model(pixel_values, output_hidden_states=True)
        feats = out.hidden_states[c.vision_feature_layer]
        if c.vision_feature_select_strategy == "default" and c.vision_config.use_class_token:
            feats = feats[:, 1:]
        return self.multi_modal_projector(feats)

    def merge_embeddings(self, input_ids, pixel_values=None, image_features=None):
        emb = self.get_input_embeddings()(input_ids)
        if pixel_values is None and image_features is None:
            return emb
        feats = image_features if image_features is not None else self.get_image_features(pixel_values)
        mask = input_ids == self.config.image_token_index
        n_slots, n_feat = int(mask.sum()), feats.shape[0] * feats.shape[1]
        if n_slots != n_feat:
            raise ValueError(f"{n_slots} image placeholder tokens for {n_feat} image feature rows")
        emb = emb.clone()
        emb[mask] = feats.reshape(-1, feats.shape[-1]).to(emb.dtype)
        return emb

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                past_key_values=None, image_features=None, **kw):
        if inputs_embeds is None:
            first = past_key_values is None or past_key_values.seq_len() == 0
            inputs_embeds = self.merge_embeddings(input_ids, pixel_values if first else None,
                                                  image_features if first else None)
        return self.language_model(inputs_embeds=inputs_embeds, attention_mask=attention_mask,
                                   position_ids=position_ids, past_key_values=past_key_values, **kw)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        call = dict(call)
        ids = call.pop("input_ids")
        emb = self.merge_embeddings(ids, call.pop("pixel_values", None), call.pop("image_features", None))
        labels = labels.masked_fill(ids == self.config.image_token_index, loss_config.ignore_index)
        call["inputs_embeds"] = emb
        return self.language_model._compute_task_loss(labels, loss_config, loss_scale, call, loss_kwargs)
