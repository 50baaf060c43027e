"""Every model type the reference's configuration files name resolves to a configuration class here, and the
composite checkpoints' halves resolve to the classes that implement them."""

import pytest

from easydel_b200.infra import factory
from easydel_b200.infra.factory import TaskType, registry

MODEL_TYPES = """
    arctic aya_vision clip clip_text_model clip_vision_model cohere dbrx deepseek_v2 deepseek_v3 exaone exaone4
    falcon falcon_h1 falcon_mamba gemma gemma2 gemma3 gemma3_text gemma4 gemma4_text gemma4_vision gidd glm glm4
    glm46v glm4_moe glm4_moe_lite glm4v glm4v_moe glm4v_moe_text glm4v_moe_vision glm4v_text glm4v_vision
    glm_moe_dsa gpt2 gpt_neox gpt_oss gptj grok-1 internlm2 kimi_linear kimi_vl llama llama4 llama4_text
    llama4_vision_model llava mamba mamba2 minimax mistral mistral3 mixtral moonvit mpt olmo olmo2 olmo3 openelm
    opt phi phi3 phimoe pixtral qwen2 qwen2_moe qwen2_vl qwen2_vl_text qwen3 qwen3_5 qwen3_5_moe
    qwen3_5_moe_text qwen3_5_text qwen3_moe qwen3_next qwen3_omni_moe qwen3_omni_moe_audio_encoder
    qwen3_omni_moe_code2wav qwen3_omni_moe_talker qwen3_omni_moe_talker_code_predictor
    qwen3_omni_moe_talker_text qwen3_omni_moe_text qwen3_omni_moe_thinker qwen3_omni_moe_vision_encoder qwen3_vl
    qwen3_vl_moe qwen3_vl_moe_text qwen3_vl_moe_vision qwen3_vl_text qwen3_vl_vision roberta rwkv seed_oss
    siglip siglip_text_model siglip_vision_model smollm3 stablelm whisper xerxes xerxes2
""".split()


def test_every_model_type_has_a_config():
    factory._ensure_models_imported()
    assert len(MODEL_TYPES) == 101
    missing = [t for t in MODEL_TYPES if t not in registry.config_registry]
    assert not missing, missing


@pytest.mark.parametrize("alias,target", [("qwen2_vl_text", "qwen2"), ("qwen3_vl_text", "qwen3"),
                                          ("qwen3_vl_moe_text", "qwen3_moe"), ("glm4v_moe_text", "glm4_moe"),
                                          ("qwen3_omni_moe_text", "qwen3_moe")])
def test_text_halves_resolve_to_their_decoder(alias, target):
    factory._ensure_models_imported()
    assert registry.get_config(alias) is registry.get_config(target)
    a = registry.get_module_registration(TaskType.CAUSAL_LM, alias)
    assert a.module is registry.get_module_registration(TaskType.CAUSAL_LM, target).module


def test_alias_of_unknown_target_raises():
    with pytest.raises(KeyError):
        registry.alias("some_alias", "no_such_model_type")
    with pytest.raises(KeyError):
        registry.get_config("no_such_model_type")


def test_llama4_composite_is_registered_for_image_text():
    factory._ensure_models_imported()
    reg = registry.get_module_registration(TaskType.IMAGE_TEXT_TO_TEXT, "llama4")
    assert reg.module.__name__ == "Llama4ForConditionalGeneration"
    assert registry.get_module_registration(TaskType.BASE_VISION, "llama4_vision_model").module.__name__ == \
        "Llama4VisionModel"
