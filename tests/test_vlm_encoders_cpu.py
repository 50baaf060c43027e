"""LLaVA (CLIP tower + projector + Llama), the SigLIP tower and RoBERTa against Hugging Face on CPU."""

import pytest
import torch
import transformers

from easydel_b200.utils.parameters_transformation import hf_to_internal, internal_to_hf

VKW = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28,
           patch_size=14)
TKW = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2)


def _jitter(model):
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)


def test_llava_matches_hf_trains_and_generates():
    from easydel_b200.modules.llava import LlavaConfig, LlavaForConditionalGeneration

    cfg = LlavaConfig(vision_config=dict(model_type="clip_vision_model", **VKW),
                      text_config=dict(model_type="llama", **TKW), image_token_index=127)
    torch.manual_seed(0)
    m = LlavaForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.LlavaForConditionalGeneration(transformers.LlavaConfig(
        vision_config=transformers.CLIPVisionConfig(**VKW), text_config=transformers.LlamaConfig(**TKW),
        image_token_index=127)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and all("position_ids" in x for x in missing), (missing, unexpected)
    ids = torch.randint(0, 120, (2, 12))
    ids[:, 2:6] = 127
    pix = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        a, b = m(input_ids=ids, pixel_values=pix).logits, hf(input_ids=ids, pixel_values=pix).logits
    assert (a - b).abs().max() < 2e-4
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_ids=ids, pixel_values=pix, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss)
    # incremental decoding: image features enter with the prompt only
    cache = m.init_cache(2, 16)
    with torch.no_grad():
        o1 = m(input_ids=ids[:, :10], pixel_values=pix, past_key_values=cache).logits
        cache.advance(10)
        o2 = m(input_ids=ids[:, 10:11], past_key_values=cache).logits
    assert (o2[:, 0] - a[:, 10]).abs().max() < 2e-4 and (o1 - a[:, :10]).abs().max() < 2e-4


def test_siglip_tower_matches_hf():
    from easydel_b200.modules.vision import SiglipVisionConfig, SiglipVisionModel

    kw = dict(VKW, patch_size=14)
    m = SiglipVisionModel(SiglipVisionConfig(**kw), dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf_cfg = transformers.SiglipVisionConfig(**kw, vision_use_head=False) if "vision_use_head" in \
        transformers.SiglipVisionConfig().to_dict() else transformers.SiglipVisionConfig(**kw)
    hf = transformers.SiglipVisionModel(hf_cfg).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and all("head" in x or "position_ids" in x for x in missing), (missing, unexpected)
    pix = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        a = m(pix).last_hidden_state
        b = hf(pixel_values=pix).last_hidden_state
    assert (a - b).abs().max() < 2e-4


def test_roberta_heads_match_hf():
    from easydel_b200.modules.roberta import RobertaConfig, RobertaForMaskedLM, RobertaForSequenceClassification

    kw = dict(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
              max_position_embeddings=40, type_vocab_size=1)
    ids = torch.randint(3, 128, (2, 12))
    ids[1, 8:] = 1
    att = (ids != 1).long()
    m = RobertaForMaskedLM(RobertaConfig(**kw), dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.RobertaForMaskedLM(transformers.RobertaConfig(**kw)).float().eval()
    sd = internal_to_hf(m)
    sd["lm_head.decoder.weight"], sd["lm_head.decoder.bias"] = sd["roberta.embeddings.word_embeddings.weight"], \
        sd["lm_head.bias"]
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    with torch.no_grad():
        a, b = m(input_ids=ids, attention_mask=att).logits, hf(input_ids=ids, attention_mask=att).logits
    assert (a - b)[att.bool()].abs().max() < 2e-3
    c = RobertaForSequenceClassification(RobertaConfig(num_labels=3, **kw), dtype=torch.float32,
                                         param_dtype=torch.float32).eval()
    hfc = transformers.RobertaForSequenceClassification(transformers.RobertaConfig(num_labels=3, **kw)).float().eval()
    missing, unexpected = hfc.load_state_dict(internal_to_hf(c), strict=False)
    assert not missing and not unexpected
    with torch.no_grad():
        assert (c(input_ids=ids, attention_mask=att).logits - hfc(input_ids=ids, attention_mask=att).logits
                ).abs().max() < 2e-3


SV = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28,
          patch_size=7)


def _check_vlm(m, hf, ids, pix, tol=3e-4):
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and all("position_ids" in x or ".head." in x or x == "lm_head.weight" for x in missing), (missing, unexpected)
    with torch.no_grad():
        a, b = m(input_ids=ids, pixel_values=pix).logits, hf(input_ids=ids, pixel_values=pix).logits
    assert (a - b).abs().max() < tol * max(1.0, float(b.abs().max())), (a - b).abs().max()
    back = hf_to_internal(m, {k: v for k, v in hf.state_dict().items() if k != "lm_head.weight" or
                              not hf.config.tie_word_embeddings})
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_ids=ids, pixel_values=pix, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss)


def test_gemma3_multimodal_matches_hf():
    from easydel_b200.modules.gemma3 import Gemma3Config, Gemma3ForConditionalGeneration

    tkw = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=8, sliding_window=16, query_pre_attn_scalar=8)
    cfg = Gemma3Config(vision_config=dict(model_type="siglip_vision_model", **SV),
                       text_config=dict(model_type="gemma3_text", **tkw), mm_tokens_per_image=4, image_token_index=127)
    torch.manual_seed(0)
    m = Gemma3ForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Gemma3ForConditionalGeneration(transformers.Gemma3Config(
        vision_config=transformers.SiglipVisionConfig(**SV), text_config=transformers.Gemma3TextConfig(**tkw),
        mm_tokens_per_image=4, image_token_index=127)).float().eval()
    ids = torch.randint(0, 120, (2, 12))
    ids[:, 2:6] = 127
    _check_vlm(m, hf, ids, torch.randn(2, 3, 28, 28))


def test_aya_vision_matches_hf():
    from easydel_b200.modules.aya_vision import AyaVisionConfig, AyaVisionForConditionalGeneration

    tkw = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, sliding_window=16, sliding_window_pattern=2, logit_scale=0.5)
    cfg = AyaVisionConfig(vision_config=dict(model_type="siglip_vision_model", **SV),
                          text_config=dict(model_type="cohere2", **tkw), downsample_factor=2, image_token_index=127)
    torch.manual_seed(0)
    m = AyaVisionForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.AyaVisionForConditionalGeneration(transformers.AyaVisionConfig(
        vision_config=transformers.SiglipVisionConfig(**SV), text_config=transformers.Cohere2Config(**tkw),
        downsample_factor=2, image_token_index=127)).float().eval()
    ids = torch.randint(0, 120, (2, 12))
    ids[:, 2:6] = 127        # 4x4 patches folded 2x2 -> 4 image tokens
    _check_vlm(m, hf, ids, torch.randn(2, 3, 28, 28))


def _dual(ours_cls, cfg_cls, hf_cls, hf_cfg_cls, extra=None, text_extra=None):
    V = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28,
             patch_size=14)
    T = dict(vocab_size=99, hidden_size=24, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
             max_position_embeddings=16, eos_token_id=98, **(text_extra or {}))
    kw = dict(extra or {})
    torch.manual_seed(0)
    m = ours_cls(cfg_cls(text_config=dict(T), vision_config=dict(V), **kw), dtype=torch.float32,
                 param_dtype=torch.float32).eval()
    _jitter(m)
    hf = hf_cls(hf_cfg_cls(text_config=dict(T), vision_config=dict(V), **kw)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and all("position_ids" in x for x in missing), (missing, unexpected)
    ids = torch.randint(0, 97, (3, 10))
    ids[:, -1] = 98
    ids[0, 6] = 98          # an earlier end-of-text token: CLIP pools there
    pix = torch.randn(3, 3, 28, 28)
    with torch.no_grad():
        a, b = m(input_ids=ids, pixel_values=pix, return_loss=True), hf(input_ids=ids, pixel_values=pix,
                                                                         return_loss=True)
    assert (a.logits_per_text - b.logits_per_text).abs().max() < 2e-4
    assert (a.image_embeds - b.image_embeds).abs().max() < 2e-5
    assert abs(float(a.loss) - float(b.loss)) < 2e-4
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())


def test_clip_dual_tower_matches_hf():
    from easydel_b200.modules.vision import CLIPConfig, CLIPModel

    _dual(CLIPModel, CLIPConfig, transformers.CLIPModel, transformers.CLIPConfig, dict(projection_dim=20))


def test_siglip_dual_tower_matches_hf():
    from easydel_b200.modules.vision import SiglipConfig, SiglipModel

    _dual(SiglipModel, SiglipConfig, transformers.SiglipModel, transformers.SiglipConfig,
          text_extra=dict(projection_size=32))


def test_mistral3_pixtral_matches_hf_with_images_of_two_sizes():
    from easydel_b200.modules.mistral3 import Mistral3Config, Mistral3ForConditionalGeneration

    V = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=56,
             patch_size=7, head_dim=8)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=8)
    cfg = Mistral3Config(vision_config=dict(model_type="pixtral", **V), text_config=dict(model_type="mistral", **T),
                         image_token_index=127, spatial_merge_size=2)
    torch.manual_seed(0)
    m = Mistral3ForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Mistral3ForConditionalGeneration(transformers.Mistral3Config(
        vision_config=transformers.PixtralVisionConfig(**V), text_config=transformers.MistralConfig(**T),
        image_token_index=127, spatial_merge_size=2, tie_word_embeddings=False)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    # image 0: 28 x 56 pixels -> 4 x 8 patches -> 2 x 4 merged rows; image 1: 56 x 28 -> 8 x 4 -> 4 x 2
    pix = torch.randn(2, 3, 56, 56)
    sizes = torch.tensor([[28, 56], [56, 28]])
    ids = torch.randint(0, 120, (1, 24))
    ids[0, 2:10] = 127
    ids[0, 12:20] = 127
    with torch.no_grad():
        a = m(input_ids=ids, pixel_values=pix, image_sizes=sizes).logits
        b = hf(input_ids=ids, pixel_values=pix, image_sizes=sizes).logits
    assert (a - b).abs().max() < 3e-4, (a - b).abs().max()
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_ids=ids, pixel_values=pix, image_sizes=sizes, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss)


def test_qwen2_vl_matches_hf_and_decodes_incrementally():
    from easydel_b200.modules.qwen2_vl import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    V = dict(depth=2, embed_dim=32, hidden_size=32, mlp_ratio=2, num_heads=4, in_channels=3, patch_size=7,
             spatial_merge_size=2, temporal_patch_size=2)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [1, 1, 2]})
    cfg = Qwen2VLConfig(vision_config=dict(V), text_config=dict(T), image_token_id=127)
    torch.manual_seed(0)
    m = Qwen2VLForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Qwen2VLForConditionalGeneration(transformers.Qwen2VLConfig(
        vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126,
        vision_start_token_id=125)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    # two images: 4 x 8 patches -> 2 x 4 = 8 tokens, and 4 x 4 patches -> 2 x 2 = 4 tokens
    grid = torch.tensor([[1, 4, 8], [1, 4, 4]])
    pix = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 7 * 7)
    ids = torch.randint(0, 120, (1, 24))
    ids[0, 2:10] = 127
    ids[0, 13:17] = 127
    with torch.no_grad():
        a = m(input_ids=ids, pixel_values=pix, image_grid_thw=grid).logits
        b = hf(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=(ids == 127).long()).logits
    assert (a - b).abs().max() < 3e-4, (a - b).abs().max()
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_ids=ids, pixel_values=pix, image_grid_thw=grid, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss)
    cache = m.init_cache(1, 32)
    with torch.no_grad():
        o1 = m(input_ids=ids[:, :20], pixel_values=pix, image_grid_thw=grid, past_key_values=cache).logits
        cache.advance(20)
        o2 = m(input_ids=ids[:, 20:21], past_key_values=cache).logits
    assert (o1 - a[:, :20]).abs().max() < 3e-4 and (o2[:, 0] - a[:, 20]).abs().max() < 3e-4


def test_qwen3_vl_deepstack_matches_hf():
    from easydel_b200.modules.qwen3_vl import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    V = dict(depth=3, hidden_size=32, intermediate_size=64, num_heads=4, in_channels=3, patch_size=7,
             spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=32, num_position_embeddings=36,
             deepstack_visual_indexes=[0, 1])
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
             num_key_value_heads=2, head_dim=8,
             rope_scaling={"rope_type": "default", "mrope_section": [2, 1, 1], "mrope_interleaved": True})
    cfg = Qwen3VLConfig(vision_config=dict(V), text_config=dict(T), image_token_id=127)
    torch.manual_seed(0)
    m = Qwen3VLForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Qwen3VLForConditionalGeneration(transformers.Qwen3VLConfig(
        vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126,
        vision_start_token_id=125)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    grid = torch.tensor([[1, 4, 8], [1, 4, 4]])
    pix = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 7 * 7)
    ids = torch.randint(0, 120, (1, 24))
    ids[0, 2:10] = 127
    ids[0, 13:17] = 127
    with torch.no_grad():
        a = m(input_ids=ids, pixel_values=pix, image_grid_thw=grid).logits
        b = hf(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=(ids == 127).long()).logits
    assert (a - b).abs().max() < 3e-4, (a - b).abs().max()
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_ids=ids, pixel_values=pix, image_grid_thw=grid, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss) and m.visual.deepstack_merger_list[0].linear_fc1.weight.grad.abs().sum() > 0


def test_qwen3_vl_moe_matches_hf():
    from easydel_b200.modules.qwen3_vl import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration
    from easydel_b200.utils.parameters_transformation import _adapt_to_hf_module_names

    V = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=4, in_channels=3, patch_size=7,
             spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=32, num_position_embeddings=36,
             deepstack_visual_indexes=[0])
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=8, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24,
             rope_scaling={"rope_type": "default", "mrope_section": [2, 1, 1], "mrope_interleaved": True})
    cfg = Qwen3VLMoeConfig(vision_config=dict(V), text_config=dict(T), image_token_id=127)
    torch.manual_seed(0)
    m = Qwen3VLMoeForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Qwen3VLMoeForConditionalGeneration(transformers.Qwen3VLMoeConfig(
        vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126,
        vision_start_token_id=125)).float().eval()
    sd = _adapt_to_hf_module_names(internal_to_hf(m), hf.state_dict())
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    grid = torch.tensor([[1, 4, 4]])
    pix = torch.randn(16, 3 * 2 * 7 * 7)
    ids = torch.randint(0, 120, (1, 12))
    ids[0, 3:7] = 127
    with torch.no_grad():
        a = m(input_ids=ids, pixel_values=pix, image_grid_thw=grid).logits
        b = hf(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=(ids == 127).long()).logits
    assert (a - b).abs().max() < 3e-4, (a - b).abs().max()


def test_glm4v_matches_hf():
    from easydel_b200.modules.glm4v import Glm4vConfig, Glm4vForConditionalGeneration

    V = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=4, in_channels=3, patch_size=7,
             spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=32, image_size=56)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2,
             rope_scaling={"rope_type": "default", "mrope_section": [1, 1, 2], "partial_rotary_factor": 1.0})
    cfg = Glm4vConfig(vision_config=dict(V), text_config=dict(T), image_token_id=127)
    torch.manual_seed(0)
    m = Glm4vForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Glm4vForConditionalGeneration(transformers.Glm4vConfig(
        vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    grid = torch.tensor([[1, 4, 8], [1, 4, 4]])
    pix = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 7 * 7)
    ids = torch.randint(0, 120, (1, 24))
    ids[0, 2:10] = 127
    ids[0, 13:17] = 127
    with torch.no_grad():
        a = m(input_ids=ids, pixel_values=pix, image_grid_thw=grid).logits
        b = hf(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=(ids == 127).long()).logits
    assert (a - b).abs().max() < 3e-4, (a - b).abs().max()
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())


def test_glm4v_moe_matches_hf():
    from easydel_b200.modules.glm4v import Glm4vMoeConfig, Glm4vMoeForConditionalGeneration
    from easydel_b200.utils.parameters_transformation import _adapt_to_hf_module_names

    V = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=4, in_channels=3, patch_size=7,
             spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=32, image_size=56)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=8, moe_intermediate_size=24, n_routed_experts=4, num_experts_per_tok=2,
             n_shared_experts=1, first_k_dense_replace=1, partial_rotary_factor=0.5, attention_bias=True,
             rope_scaling={"rope_type": "default", "mrope_section": [1, 1]}, pad_token_id=0)
    cfg = Glm4vMoeConfig(vision_config=dict(V), text_config=dict(T), image_token_id=127)
    torch.manual_seed(0)
    m = Glm4vMoeForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Glm4vMoeForConditionalGeneration(transformers.Glm4vMoeConfig(
        vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126)).float().eval()
    sd = _adapt_to_hf_module_names(internal_to_hf(m), hf.state_dict())
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    grid = torch.tensor([[1, 4, 4]])
    pix = torch.randn(16, 3 * 2 * 7 * 7)
    ids = torch.randint(1, 120, (1, 12))
    ids[0, 3:7] = 127
    with torch.no_grad():
        a = m(input_ids=ids, pixel_values=pix, image_grid_thw=grid).logits
        b = hf(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=(ids == 127).long()).logits
    assert (a - b).abs().max() < 3e-4, (a - b).abs().max()


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_5_hybrid_vlm_matches_hf(moe):
    from easydel_b200.modules.qwen3_vl import (Qwen3_5Config, Qwen3_5ForConditionalGeneration, Qwen3_5MoeConfig,
                                               Qwen3_5MoeForConditionalGeneration)
    from easydel_b200.utils.parameters_transformation import _adapt_to_hf_module_names

    V = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=4, in_channels=3, patch_size=7,
             spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=32, num_position_embeddings=36)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
             num_key_value_heads=2, head_dim=16, linear_num_value_heads=4, linear_num_key_heads=2,
             linear_key_head_dim=8, linear_value_head_dim=16,
             layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
             rope_parameters=dict(rope_type="default", rope_theta=1e6, partial_rotary_factor=0.5,
                                  mrope_section=[2, 1, 1], mrope_interleaved=True))
    if moe:
        T.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24, shared_expert_intermediate_size=48)
    ours_cfg, ours_cls = (Qwen3_5MoeConfig, Qwen3_5MoeForConditionalGeneration) if moe else \
        (Qwen3_5Config, Qwen3_5ForConditionalGeneration)
    hf_cfg_cls, hf_cls = (transformers.Qwen3_5MoeConfig, transformers.Qwen3_5MoeForConditionalGeneration) if moe \
        else (transformers.Qwen3_5Config, transformers.Qwen3_5ForConditionalGeneration)
    torch.manual_seed(0)
    hf = hf_cls(hf_cfg_cls(vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126,
                           vision_start_token_id=125)).float().eval()
    m = ours_cls(ours_cfg(vision_config=dict(V), text_config=dict(T), image_token_id=127), dtype=torch.float32,
                 param_dtype=torch.float32).eval()
    m.load_state_dict(hf_to_internal(m, hf.state_dict()))
    grid = torch.tensor([[1, 4, 4]])
    pix = torch.randn(16, 3 * 2 * 7 * 7)
    ids = torch.randint(0, 120, (1, 14))
    ids[0, 3:7] = 127
    with torch.no_grad():
        a = m(input_ids=ids, pixel_values=pix, image_grid_thw=grid).logits
        b = hf(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=(ids == 127).long()).logits
    assert (a - b).abs().max() < 3e-4, (a - b).abs().max()
    sd = _adapt_to_hf_module_names(internal_to_hf(m), hf.state_dict())
    assert set(sd) == set(hf.state_dict())


def test_qwen2_vl_video_matches_hf():
    from easydel_b200.modules.qwen2_vl import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    V = dict(depth=2, embed_dim=32, hidden_size=32, num_heads=4, in_channels=3, patch_size=7, spatial_merge_size=2,
             temporal_patch_size=2, mlp_ratio=2)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [1, 1, 2]})
    torch.manual_seed(0)
    hf = transformers.Qwen2VLForConditionalGeneration(transformers.Qwen2VLConfig(
        vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126,
        vision_start_token_id=125)).float().eval()
    m = Qwen2VLForConditionalGeneration(Qwen2VLConfig(vision_config=dict(V), text_config=dict(T), image_token_id=127,
                                                      video_token_id=126), dtype=torch.float32,
                                        param_dtype=torch.float32).eval()
    m.load_state_dict(hf_to_internal(m, hf.state_dict()))
    vgrid = torch.tensor([[2, 4, 4]])                 # two temporal patches of a 4 x 4 patch grid -> 8 tokens
    vpix = torch.randn(32, 3 * 2 * 7 * 7)
    igrid = torch.tensor([[1, 4, 4]])
    ipix = torch.randn(16, 3 * 2 * 7 * 7)
    ids = torch.randint(0, 120, (1, 26))
    ids[0, 2:10] = 126
    ids[0, 14:18] = 127
    kw = dict(input_ids=ids, pixel_values=ipix, image_grid_thw=igrid, pixel_values_videos=vpix, video_grid_thw=vgrid)
    with torch.no_grad():
        a = m(**kw).logits
        b = hf(mm_token_type_ids=(ids == 127).long() + 2 * (ids == 126).long(), **kw).logits
    assert (a - b).abs().max() < 1e-3, (a - b).abs().max()
    _, met = m.compute_loss(labels=ids, **kw)
    assert torch.isfinite(met.loss)


def test_qwen3_vl_video_frames_match_hf():
    from easydel_b200.modules.qwen3_vl import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    V = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=4, in_channels=3, patch_size=7,
             spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=32, num_position_embeddings=36,
             deepstack_visual_indexes=[0])
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=8,
             rope_scaling={"rope_type": "default", "mrope_section": [2, 1, 1], "mrope_interleaved": True})
    torch.manual_seed(0)
    hf = transformers.Qwen3VLForConditionalGeneration(transformers.Qwen3VLConfig(
        vision_config=dict(V), text_config=dict(T), image_token_id=127, video_token_id=126,
        vision_start_token_id=125)).float().eval()
    m = Qwen3VLForConditionalGeneration(Qwen3VLConfig(vision_config=dict(V), text_config=dict(T), image_token_id=127,
                                                      video_token_id=126), dtype=torch.float32,
                                        param_dtype=torch.float32).eval()
    m.load_state_dict(hf_to_internal(m, hf.state_dict()))
    vgrid = torch.tensor([[2, 4, 4]])
    vpix = torch.randn(32, 3 * 2 * 7 * 7)
    ids = torch.randint(0, 120, (1, 20))
    ids[0, 3:7] = 126          # first frame group
    ids[0, 9:13] = 126         # second one, after its timestamp text
    kw = dict(input_ids=ids, pixel_values_videos=vpix, video_grid_thw=vgrid)
    with torch.no_grad():
        a = m(**kw).logits
        b = hf(mm_token_type_ids=2 * (ids == 126).long(), **kw).logits
    assert (a - b).abs().max() < 1e-3, (a - b).abs().max()


L4V = dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=128, image_size=28,
           patch_size=7, vision_output_dim=48, projector_input_dim=48, projector_output_dim=48,
           pixel_shuffle_ratio=0.5)
L4T = dict(vocab_size=128, hidden_size=32, intermediate_size=48, intermediate_size_mlp=96, num_hidden_layers=4,
           num_attention_heads=2, num_key_value_heads=1, head_dim=16, num_local_experts=4, num_experts_per_tok=1,
           attention_chunk_size=32, floor_scale=16, attn_scale=0.3, no_rope_layers=[1, 1, 1, 0],
           moe_layers=[0, 2, 3], max_position_embeddings=64, rope_theta=10000.0,
           layer_types=["chunked_attention", "chunked_attention", "chunked_attention", "full_attention"])


def test_llama4_vision_tower_matches_hf():
    from easydel_b200.modules.llama4 import Llama4VisionConfig, Llama4VisionModel, pixel_shuffle

    torch.manual_seed(0)
    m = Llama4VisionModel(Llama4VisionConfig(**L4V), dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf = transformers.Llama4VisionModel(transformers.Llama4VisionConfig(
        **L4V, rope_parameters=dict(rope_theta=10000.0, rope_type="default"))).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not missing and not unexpected
    pix = torch.randn(3, 3, 28, 28)
    with torch.no_grad():
        a, b = m(pix).last_hidden_state, hf(pix).last_hidden_state
    assert a.shape == (3, 4, 48) and (a - b).abs().max() < 1e-5          # 16 patches fold into 4 rows
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    # the shuffle folds a 2 x 2 neighbourhood of the grid into the channel axis
    grid = torch.arange(16.0).view(1, 16, 1).expand(1, 16, 2).contiguous()
    out = pixel_shuffle(grid, 0.5)
    assert out.shape == (1, 4, 8) and sorted(out[0, 0, ::2].tolist()) == [0.0, 1.0, 4.0, 5.0]


def test_llama4_multimodal_matches_hf_trains_and_decodes():
    from easydel_b200.modules.llama4 import Llama4Config, Llama4ForConditionalGeneration

    cfg = Llama4Config(vision_config=dict(L4V), text_config=dict(L4T), image_token_index=127)
    assert cfg.vision_config.model_type == "llama4_vision_model" and cfg.text_config.model_type == "llama4_text"
    torch.manual_seed(0)
    m = Llama4ForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    _jitter(m)
    hf_cfg = transformers.Llama4Config(
        vision_config=dict(L4V, rope_parameters=dict(rope_theta=10000.0, rope_type="default")),
        text_config=dict({k: v for k, v in L4T.items() if k != "rope_theta"},
                         rope_parameters=dict(rope_theta=10000.0, rope_type="default")),
        image_token_index=127)
    hf_cfg._attn_implementation = "eager"
    hf = transformers.Llama4ForConditionalGeneration(hf_cfg).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    ids = torch.randint(0, 120, (2, 14))
    ids[:, 2:6] = 127                                              # one tile -> four feature rows per sequence
    pix = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        a, b = m(input_ids=ids, pixel_values=pix).logits, hf(input_ids=ids, pixel_values=pix).logits
        t1, t2 = m(input_ids=ids).logits, hf(input_ids=ids).logits
    assert (t1 - t2).abs().max() < 3e-4 and (a - b).abs().max() < 3e-4
    assert (a - t1).abs().max() > 1e-3                             # the image changed something
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_ids=ids, pixel_values=pix, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss) and m.vision_model.patch_embedding.linear.weight.grad.abs().sum() > 0
    cache = m.init_cache(2, 16)
    with torch.no_grad():
        o1 = m(input_ids=ids[:, :10], pixel_values=pix, past_key_values=cache).logits
        cache.advance(10)
        o2 = m(input_ids=ids[:, 10:11], past_key_values=cache).logits
    assert (o2[:, 0] - a[:, 10]).abs().max() < 3e-4 and (o1 - a[:, :10]).abs().max() < 3e-4
    with pytest.raises(ValueError):                                # placeholders and feature rows must agree
        m(input_ids=ids[:, :4], pixel_values=pix)
