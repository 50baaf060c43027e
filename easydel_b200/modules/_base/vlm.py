"""Shared machinery of the vision-language models: a vision tower, a projector and a causal language model whose
placeholder-token embeddings are overwritten with projected image features (easydel/infra/mixins and the
``BaseVisionLanguageModule`` of easydel/modules/_base).

Subclasses define the projector, ``get_image_features`` and the weight-name tables. After the merge everything is the
text model, so training, generation and serving reuse the decoder path through ``inputs_embeds``.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, registry
from ...infra.loss_utils import LossConfig
from .families import _Renamer


def build_sub_config(c, default_type: str):
    if c is None:
        c = {}
    if isinstance(c, dict):
        c = dict(c)
        return registry.get_config(c.pop("model_type", default_type))(**c)
    return c


class VLMConfig(EasyDeLBaseConfig):
    """``vision_config`` + ``text_config`` (dicts or config objects) + the placeholder token id."""

    vision_default, text_default = "clip_vision_model", "llama"

    def __init__(self, **kw):   # explicit: the config base class generates a constructor for classes without one
        super().__init__(**kw)

    def _init_parts(self, vision_config, text_config, image_token_index, kw):
        self.vision_config = build_sub_config(vision_config, self.vision_default)
        self.text_config = build_sub_config(text_config, self.text_default)
        self.image_token_index = image_token_index
        for k in ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads"):
            setattr(self, k, getattr(self.text_config, k, None))
        kw.setdefault("tie_word_embeddings", getattr(self.text_config, "tie_word_embeddings", False))
        return kw

    def to_dict(self):
        d = super().to_dict()
        d["vision_config"] = self.vision_config.to_dict()
        d["text_config"] = self.text_config.to_dict()
        return d


class VisionTower(nn.Module):
    def __init__(self, cfg, dtype):
        super().__init__()
        from ..vision.vit import VisionTransformer

        self.vision_model = VisionTransformer(cfg, dtype)


OUTER_RULES = [("model.vision_tower.", "vision_tower."), ("model.multi_modal_projector.", "multi_modal_projector."),
               ("model.language_model.", "language_model.model."), ("lm_head.", "language_model.lm_head.")]


class VLMForConditionalGeneration(EasyDeLBaseModule):
    loss_type = "ForCausalLM"
    hf_keeps_fused = ()
    outer_rules = OUTER_RULES
    # checkpoint tensors that have no counterpart here (e.g. the pooling head of a SigLIP tower)
    ignored_prefixes: tuple[str, ...] = ("model.vision_tower.vision_model.head.", "vision_tower.vision_model.head.")

    def build_language_model(self, config, dtype, param_dtype, precision, rngs):
        reg = registry.get_module_registration(TaskType.CAUSAL_LM, config.text_config.model_type)
        return reg.module(config.text_config, dtype, param_dtype, precision, rngs)

    # ------------------------------------------------------------------ weight names
    def _vision_renamer(self):
        from ..vision.vit import VISION_RULES

        return _Renamer(VISION_RULES)

    def hf_rename_in(self, sd):
        sd = {k: v for k, v in sd.items() if not k.endswith("position_ids")
              and not any(k.startswith(p) for p in self.ignored_prefixes)}
        outer = _Renamer(self.outer_rules)
        vis = {k: v for k, v in sd.items() if ".vision_tower." in k or k.startswith("vision_tower.")}
        rest = {k: v for k, v in sd.items() if k not in vis}
        lm_in = getattr(self.language_model, "hf_rename_in", None)
        out = outer.to_internal(self, rest)
        if lm_in is not None:     # the language model's own table, applied under its prefix
            lm = {k[len("language_model."):]: v for k, v in out.items() if k.startswith("language_model.")}
            out = {k: v for k, v in out.items() if not k.startswith("language_model.")}
            out.update({"language_model." + k: v for k, v in lm_in(lm).items()})
        out.update(outer.to_internal(self, self._vision_renamer().to_internal(self, vis)))
        return out

    def hf_rename_out(self, sd):
        outer = _Renamer(self.outer_rules)
        vis = {k: v for k, v in sd.items() if k.startswith("vision_tower.")}
        rest = {k: v for k, v in sd.items() if k not in vis}
        lm_out = getattr(self.language_model, "hf_rename_out", None)
        if lm_out is not None:
            lm = {k[len("language_model."):]: v for k, v in rest.items() if k.startswith("language_model.")}
            rest = {k: v for k, v in rest.items() if not k.startswith("language_model.")}
            rest.update({"language_model." + k: v for k, v in lm_out(lm).items()})
        out = outer.to_hf(self, rest)
        out.update(outer.to_hf(self, self._vision_renamer().to_hf(self, vis)))
        return out

    # ------------------------------------------------------------------ language-model facade
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

    # ------------------------------------------------------------------ merge + forward
    def get_image_features(self, pixel_values: torch.Tensor, **kw) -> torch.Tensor:
        raise NotImplementedError

    def embed_text(self, input_ids):
        """Token embeddings as the language model's first layer sees them before its own scaling."""
        return self.get_input_embeddings()(input_ids)

    def merge_embeddings(self, input_ids, pixel_values=None, image_features=None, **kw):
        emb = self.embed_text(input_ids)
        if pixel_values is None and image_features is None:
            return emb
        feats = image_features if image_features is not None else self.get_image_features(pixel_values, **kw)
        mask = input_ids == self.config.image_token_index
        n_slots, n_feat = int(mask.sum()), feats.numel() // feats.shape[-1]
        if n_slots != n_feat:
            raise ValueError(f"{n_slots} image placeholder tokens for {n_feat} image feature rows")
        emb = emb.clone()
        emb[mask] = feats.reshape(-1, feats.shape[-1]).to(emb.dtype)
        return emb

    image_kwargs: tuple[str, ...] = ()

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                past_key_values=None, image_features=None, **kw):
        extra = {k: kw.pop(k) for k in self.image_kwargs if k in kw}
        if inputs_embeds is None:
            first = past_key_values is None or past_key_values.seq_len() == 0
            inputs_embeds = self.merge_embeddings(input_ids, pixel_values if first else None,
                                                  image_features if first else None, **extra)
        return self.language_model(inputs_embeds=inputs_embeds, attention_mask=attention_mask,
                                   position_ids=position_ids, past_key_values=past_key_values, **kw)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        call = dict(call)
        ids = call.pop("input_ids")
        extra = {k: call.pop(k) for k in self.image_kwargs if k in call}
        emb = self.merge_embeddings(ids, call.pop("pixel_values", None), call.pop("image_features", None), **extra)
        labels = labels.masked_fill(ids == self.config.image_token_index, loss_config.ignore_index)
        call["inputs_embeds"] = emb
        return self.language_model._compute_task_loss(labels, loss_config, loss_scale, call, loss_kwargs)
