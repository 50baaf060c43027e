"""Names of the flat public namespace that are built from existing classes: other spellings, the halves of composite
models, head-less multimodal models, added classification heads and the embedding models."""

import pytest
import torch

import easydel_b200 as ed
from easydel_b200.infra.factory import TaskType, registry

TKW = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2)
VKW = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28,
           patch_size=14)


@pytest.mark.parametrize("name", [
    "PhiMoeConfig", "PhiMoeModel", "PhiMoeForCausalLM", "StableLmConfig", "StableLmModel", "StableLmForCausalLM",
    "GPT2LMHeadModel", "Llama4ForCausalLM", "Llama4ForSequenceClassification", "Llama4ForConditionalGeneration",
    "Llama4VisionModel", "Gemma3ForCausalLM", "Gemma3ForSequenceClassification", "Qwen3_5ForCausalLM",
    "Qwen3_5MoeForCausalLM", "Qwen3VLTextConfig", "Qwen3VLTextModel", "Qwen3VLMoeTextConfig", "Qwen3VLMoeTextModel",
    "Qwen3VLMoeVisionConfig", "Qwen3VisionTransformerPretrainedModel", "Qwen3VLMoeVisionTransformerPretrainedModel",
    "Qwen3OmniMoeTextConfig", "Qwen3OmniMoeVisionConfig", "Qwen3OmniMoeVisionEncoderConfig",
    "Qwen3OmniMoeVisionEncoder", "Qwen3OmniMoeAudioConfig", "Qwen3OmniMoeTalkerCodePredictorForConditionalGeneration",
    "Qwen3OmniMoeTalkerCodePredictorModel", "Qwen3_5MoeVisionConfig", "Glm4vMoeTextConfig", "Glm4vMoeTextModel",
    "Glm4vMoeVisionConfig", "Glm4vVisionModel", "Glm4vMoeVisionModel", "LlavaModel", "AyaVisionModel",
    "Mistral3Model", "Qwen2VLModel", "Qwen3VLModel", "Qwen3VLMoeModel", "Glm4vModel", "Glm46VModel", "Glm4vMoeModel",
    "Qwen3_5Model", "Qwen3_5MoeModel", "Qwen3OmniMoeThinkerModel", "Qwen3OmniMoeModel",
    "DbrxForSequenceClassification", "Glm4MoeForSequenceClassification", "Qwen2ForEmbedding", "Qwen3ForEmbedding",
    "EasyDeLRuntimeError", "EasyDeLSyntaxRuntimeError", "EasyDeLTimerError", "EasyDeLBackends", "EasyDeLPlatforms",
    "MoEMethods", "Registry", "ModelConverter", "StateDictConverter", "TensorConverter", "ToolParser",
    "EngineRequest", "EngineRequestStatus", "ResponsesStreamBuilder"])
def test_name_resolves_to_a_class(name):
    assert isinstance(getattr(ed, name), type)


def test_headless_multimodal_model_returns_the_full_models_hidden_states():
    cfg = ed.LlavaConfig(vision_config=dict(model_type="clip_vision_model", **VKW),
                         text_config=dict(model_type="llama", **TKW), image_token_index=127)
    torch.manual_seed(0)
    full = ed.LlavaForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    base = ed.LlavaModel(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    base.load_state_dict(full.state_dict())
    ids = torch.randint(0, 120, (2, 12))
    ids[:, 2:6] = 127
    pix = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        want = full(input_ids=ids, pixel_values=pix)
        got = base(input_ids=ids, pixel_values=pix)
    assert not hasattr(got, "logits") and torch.equal(got.last_hidden_state, want.last_hidden_state)
    assert not base.can_generate() and full.can_generate()
    assert registry.get_module_registration(TaskType.BASE_MODULE, "llava").module is ed.LlavaModel
    # the generation model is still what the image-text task resolves to
    assert registry.get_module_registration(TaskType.IMAGE_TEXT_TO_TEXT, "llava").module is \
        ed.LlavaForConditionalGeneration


def test_embedding_model_pools_and_normalises():
    cfg = ed.Qwen3Config(**TKW, head_dim=8)
    torch.manual_seed(0)
    m = ed.Qwen3ForEmbedding(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    ids = torch.randint(3, 120, (3, 9))
    mask = torch.ones(3, 9, dtype=torch.long)
    mask[1, 6:] = 0
    with torch.no_grad():
        out = m(input_ids=ids, attention_mask=mask)
        raw = m(input_ids=ids, attention_mask=mask, normalize=False).embeddings
    assert out.embeddings.shape == (3, 32) and torch.allclose(out.embeddings.norm(dim=-1), torch.ones(3), atol=1e-5)
    assert torch.allclose(raw[1], out.last_hidden_state[1, 5], atol=1e-6)       # last attended token
    assert torch.allclose(raw[0], out.last_hidden_state[0, 8], atol=1e-6)
    cfg.embedding_pooling = "mean"
    with torch.no_grad():
        mean = m(input_ids=ids, attention_mask=mask, normalize=False).embeddings
    assert torch.allclose(mean[1], out.last_hidden_state[1, :6].mean(0), atol=1e-5)
    assert registry.get_module_registration(TaskType.EMBEDDING, "qwen3").module is ed.Qwen3ForEmbedding
    # the backbone's weights load from the causal model's state
    lm = ed.Qwen3ForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    missing, unexpected = m.load_state_dict(lm.state_dict(), strict=False)
    assert not missing and all(k.startswith("lm_head") for k in unexpected)


def test_added_classifier_head_runs_and_trains():
    reg = registry.get_module_registration(TaskType.SEQUENCE_CLASSIFICATION, "glm4_moe")
    assert reg.module is ed.Glm4MoeForSequenceClassification
    cfg = ed.Glm4MoeConfig(**TKW, head_dim=8, moe_intermediate_size=16, n_routed_experts=4, num_experts_per_tok=2,
                           n_shared_experts=1, first_k_dense_replace=1, num_labels=3, pad_token_id=0)
    torch.manual_seed(0)
    m = reg.module(cfg, dtype=torch.float32, param_dtype=torch.float32)
    ids = torch.randint(3, 120, (2, 7))
    out = m(input_ids=ids)
    assert out.logits.shape == (2, 3)
    _, met = m.compute_loss(input_ids=ids, labels=torch.tensor([0, 2]))
    met.loss.backward()
    assert torch.isfinite(met.loss) and m.score.weight.grad.abs().sum() > 0


def test_request_status_alias():
    assert ed.EngineRequestStatus.RUNNING.value == "running" and ed.EngineRequestStatus.FINISHED_LENGTH.finished
