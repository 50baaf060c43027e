"""The remaining public class names of the reference's flat namespace (easydel/__init__.py), built from classes that
already exist here:

* spellings that differ (``PhiMoe*``, ``StableLm*``, ``GPT2LMHeadModel``) and the language / vision halves of
  composite models under the names their checkpoints' configs use (``Qwen3VLTextModel``, ``Glm4vMoeVisionConfig``...);
* head-less base models of the vision-language families (``LlavaModel``, ``Qwen2VLModel``...): the conditional
  generation model with the LM head left out of ``forward``, registered under ``TaskType.BASE_MODULE``;
* sequence-classification heads for two families whose definitions did not ask for one;
* embedding models (``Qwen2ForEmbedding``, ``Qwen3ForEmbedding``): backbone, pooling over the attention mask and an
  L2 normalisation, registered under ``TaskType.EMBEDDING``.
"""

from __future__ import annotations

import torch

from ..infra.base_module import EasyDeLBaseModule
from ..infra.factory import TaskType, register_module, registry
from ..infra.modeling_outputs import BaseModelOutput, EmbeddingOutput
from . import families, families_classic, families_extra  # noqa: F401
from ._base.decoder import DecoderForSequenceClassification
from .aya_vision import AyaVisionForConditionalGeneration
from .gemma3 import Gemma3ForConditionalGeneration
from .glm4v import (Glm4vForConditionalGeneration, Glm4vMoeForConditionalGeneration, Glm4vVisionConfig,
                    Glm4vVisionTransformer, Glm46VForConditionalGeneration)
from .llava import LlavaForConditionalGeneration
from .mistral3 import Mistral3ForConditionalGeneration
from .qwen2_vl import Qwen2VLForConditionalGeneration
from .qwen3_omni_moe import (Qwen3OmniMoeAudioEncoderConfig, Qwen3OmniMoeTalkerCodePredictor,
                             Qwen3OmniMoeThinkerForConditionalGeneration)
from .qwen3_omni_moe import speech as _speech
from .qwen3_vl import (Qwen3_5ForConditionalGeneration, Qwen3_5MoeForConditionalGeneration, Qwen3_5VisionConfig,
                       Qwen3VLForConditionalGeneration, Qwen3VLMoeForConditionalGeneration, Qwen3VLVisionConfig,
                       Qwen3VLVisionTransformer)

_F = {**families.EXPORTS, **getattr(families_classic, "EXPORTS", {}), **getattr(families_extra, "EXPORTS", {})}

EXPORTS: dict[str, type] = {}

# ---------------------------------------------------------------------------------------------- other spellings
for _new, _old in {
    "PhiMoeConfig": "PhimoeConfig", "PhiMoeModel": "PhimoeModel", "PhiMoeForCausalLM": "PhimoeForCausalLM",
    "StableLmConfig": "StablelmConfig", "StableLmModel": "StablelmModel", "StableLmForCausalLM": "StablelmForCausalLM",
    "GPT2LMHeadModel": "GPT2ForCausalLM",
    "Llama4ForCausalLM": "Llama4TextForCausalLM", "Llama4ForSequenceClassification": "Llama4TextForSequenceClassification",
    "Gemma3ForCausalLM": "Gemma3TextForCausalLM", "Gemma3ForSequenceClassification": "Gemma3TextForSequenceClassification",
    "Qwen3_5ForCausalLM": "Qwen3_5TextForCausalLM", "Qwen3_5MoeForCausalLM": "Qwen3_5MoeTextForCausalLM",
    "Qwen3VLTextConfig": "Qwen3Config", "Qwen3VLTextModel": "Qwen3Model",
    "Qwen3VLMoeTextConfig": "Qwen3MoeConfig", "Qwen3VLMoeTextModel": "Qwen3MoeModel",
    "Qwen3OmniMoeTextConfig": "Qwen3MoeConfig",
    "Glm4vMoeTextConfig": "Glm4MoeConfig", "Glm4vMoeTextModel": "Glm4MoeModel",
}.items():
    if _old in _F:
        EXPORTS[_new] = _F[_old]

EXPORTS.update(
    Glm4vMoeVisionConfig=Glm4vVisionConfig, Glm4vVisionModel=Glm4vVisionTransformer,
    Glm4vMoeVisionModel=Glm4vVisionTransformer,
    Qwen3VLMoeVisionConfig=Qwen3VLVisionConfig, Qwen3VisionTransformerPretrainedModel=Qwen3VLVisionTransformer,
    Qwen3VLMoeVisionTransformerPretrainedModel=Qwen3VLVisionTransformer,
    Qwen3OmniMoeVisionConfig=Qwen3VLVisionConfig, Qwen3OmniMoeVisionEncoderConfig=Qwen3VLVisionConfig,
    Qwen3OmniMoeVisionEncoder=Qwen3VLVisionTransformer, Qwen3OmniMoeAudioConfig=Qwen3OmniMoeAudioEncoderConfig,
    Qwen3OmniMoeTalkerCodePredictorForConditionalGeneration=Qwen3OmniMoeTalkerCodePredictor,
    Qwen3OmniMoeTalkerCodePredictorModel=_speech._PRED["Qwen3OmniMoeTalkerCodePredictorModel"],
    Qwen3_5MoeVisionConfig=Qwen3_5VisionConfig,
)


# ---------------------------------------------------------------------------------- head-less multimodal models
def _base_model(name: str, full: type, model_type: str) -> type:
    def forward(self, *args, **kw):
        kw["apply_lm_head"] = False
        out = full.forward(self, *args, **kw)
        return BaseModelOutput(last_hidden_state=out.last_hidden_state, hidden_states=out.hidden_states,
                               past_key_values=out.past_key_values)

    cls = type(name, (full,), {"forward": forward, "can_generate": lambda self: False, "__doc__":
               f"``{full.__name__}`` without the LM head: ``forward`` returns the final hidden states."})
    return register_module(TaskType.BASE_MODULE, config=full.config_class, model_type=model_type)(cls)


for _name, _full, _type in [
    ("LlavaModel", LlavaForConditionalGeneration, "llava"),
    ("AyaVisionModel", AyaVisionForConditionalGeneration, "aya_vision"),
    ("Mistral3Model", Mistral3ForConditionalGeneration, "mistral3"),
    ("Gemma3Model", Gemma3ForConditionalGeneration, "gemma3"),
    ("Qwen2VLModel", Qwen2VLForConditionalGeneration, "qwen2_vl"),
    ("Qwen3VLModel", Qwen3VLForConditionalGeneration, "qwen3_vl"),
    ("Qwen3VLMoeModel", Qwen3VLMoeForConditionalGeneration, "qwen3_vl_moe"),
    ("Glm4vModel", Glm4vForConditionalGeneration, "glm4v"),
    ("Glm46VModel", Glm46VForConditionalGeneration, "glm46v"),
    ("Glm4vMoeModel", Glm4vMoeForConditionalGeneration, "glm4v_moe"),
    ("Qwen3_5Model", Qwen3_5ForConditionalGeneration, "qwen3_5"),
    ("Qwen3_5MoeModel", Qwen3_5MoeForConditionalGeneration, "qwen3_5_moe"),
    ("Qwen3OmniMoeThinkerModel", Qwen3OmniMoeThinkerForConditionalGeneration, "qwen3_omni_moe_thinker"),
]:
    EXPORTS[_name] = _base_model(_name, _full, _type)
EXPORTS["Qwen3OmniMoeModel"] = EXPORTS["Qwen3OmniMoeThinkerModel"]


# ------------------------------------------------------------------------------------------ classification heads
def _classifier(prefix: str, model_type: str) -> type | None:
    lm, model = _F.get(prefix + "ForCausalLM"), _F.get(prefix + "Model")
    if lm is None or model is None:
        return None
    ns = {"backbone_cls": model, "hf_keeps_fused": getattr(lm, "hf_keeps_fused", ())}
    for hook in ("hf_rename_in", "hf_rename_out"):
        if hook in lm.__dict__:
            ns[hook] = lm.__dict__[hook]
    cls = type(prefix + "ForSequenceClassification", (DecoderForSequenceClassification,), ns)
    return register_module(TaskType.SEQUENCE_CLASSIFICATION, config=lm.config_class, model_type=model_type)(cls)


for _prefix, _type in [("Dbrx", "dbrx"), ("Glm4Moe", "glm4_moe")]:
    _cls = _classifier(_prefix, _type)
    if _cls is not None:
        EXPORTS[_cls.__name__] = _cls


# ---------------------------------------------------------------------------------------------- embedding models
class DecoderForEmbedding(EasyDeLBaseModule):
    """Sentence embeddings from a decoder: the backbone's final hidden states pooled over the attention mask
    (``config.embedding_pooling``: ``last`` (default), ``mean`` or ``cls``) and L2-normalised."""

    backbone_cls: type = None
    loss_type = "ForCausalLM"

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.model = type(self).backbone_cls(config, dtype, param_dtype, precision, rngs)

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, inputs_embeds=None, normalize=True, **_):
        from ..trainers.embedding import pool_hidden

        h = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                       inputs_embeds=inputs_embeds).last_hidden_state
        if attention_mask is None:
            attention_mask = torch.ones(h.shape[:2], dtype=torch.long, device=h.device)
        e = pool_hidden(h, attention_mask, getattr(self.config, "embedding_pooling", "last")).float()
        if normalize:
            e = torch.nn.functional.normalize(e, dim=-1)
        return EmbeddingOutput(embeddings=e, last_hidden_state=h)


for _prefix, _type in [("Qwen2", "qwen2"), ("Qwen3", "qwen3"), ("Llama", "llama"), ("Mistral", "mistral")]:
    _model = _F.get(_prefix + "Model")
    _lm = _F.get(_prefix + "ForCausalLM")
    if _model is None and _prefix == "Llama":
        from .llama import LlamaForCausalLM as _lm, LlamaModel as _model
    if _model is None:
        continue
    _ns = {"backbone_cls": _model, "hf_keeps_fused": getattr(_lm, "hf_keeps_fused", ())}
    for _hook in ("hf_rename_in", "hf_rename_out"):
        if _lm is not None and _hook in _lm.__dict__:
            _ns[_hook] = _lm.__dict__[_hook]
    _cls = type(_prefix + "ForEmbedding", (DecoderForEmbedding,), _ns)
    EXPORTS[_cls.__name__] = register_module(TaskType.EMBEDDING, config=registry.get_config(_type),
                                             model_type=_type)(_cls)

globals().update(EXPORTS)
__all__ = sorted(EXPORTS) + ["DecoderForEmbedding"]
