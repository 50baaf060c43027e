"""Qwen3-Omni-MoE thinker against Hugging Face: audio tower alone, then text + image + audio through the model."""

import torch
from transformers.models.qwen3_omni_moe import configuration_qwen3_omni_moe as hc
from transformers.models.qwen3_omni_moe import modeling_qwen3_omni_moe as hm

from easydel_b200.modules.qwen3_omni_moe import (Qwen3OmniMoeConfig, Qwen3OmniMoeForConditionalGeneration,
                                                 Qwen3OmniMoeThinkerConfig,
                                                 Qwen3OmniMoeThinkerForConditionalGeneration, audio_output_lengths)
from easydel_b200.utils.parameters_transformation import _adapt_to_hf_module_names, hf_to_internal, internal_to_hf

A = dict(num_mel_bins=16, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=48, d_model=32, n_window=8,
         output_dim=48, n_window_infer=32, downsample_hidden_size=8, max_source_positions=64)
V = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, patch_size=4, out_hidden_size=48,
         num_position_embeddings=16, deepstack_visual_indexes=[0])
T = dict(vocab_size=200, hidden_size=48, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
         num_key_value_heads=2, head_dim=16, moe_intermediate_size=24, num_experts_per_tok=2, num_experts=4,
         rope_parameters=dict(rope_type="default", rope_theta=1e6, mrope_section=[2, 3, 3], mrope_interleaved=True))
IDS = dict(audio_token_id=190, image_token_id=191, video_token_id=192, audio_start_token_id=193)


def _pair():
    torch.manual_seed(0)
    hcfg = hc.Qwen3OmniMoeThinkerConfig(audio_config=dict(A), vision_config=dict(V), text_config=dict(T),
                                        vision_start_token_id=194, vision_end_token_id=195, **IDS)
    hcfg._attn_implementation = "eager"
    for sub in (hcfg.audio_config, hcfg.vision_config, hcfg.text_config):
        sub._attn_implementation = "eager"
    hf = hm.Qwen3OmniMoeThinkerForConditionalGeneration(hcfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)
    cfg = Qwen3OmniMoeThinkerConfig(audio_config=dict(A), vision_config=dict(V), text_config=dict(T), **IDS)
    m = Qwen3OmniMoeThinkerForConditionalGeneration(cfg, dtype=torch.float32).eval()
    m.load_state_dict(hf_to_internal(m, hf.state_dict()))
    return hf, m


def test_audio_tower_matches_hf_over_clips_of_unequal_length():
    hf, m = _pair()
    lens = torch.tensor([37, 16, 50])
    assert audio_output_lengths(lens).tolist() == hm._get_feat_extract_output_lengths(lens).tolist()
    feats = torch.randn(16, int(lens.sum()))
    with torch.no_grad():
        want = hf.audio_tower(feats, feature_lens=lens).last_hidden_state
        got = m.audio_tower(feats, lens)
    assert got.shape == (int(audio_output_lengths(lens).sum()), 48)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)


def test_thinker_matches_hf_with_image_and_audio_then_decodes_and_trains():
    hf, m = _pair()
    frames = torch.tensor([37, 22])
    n_audio = audio_output_lengths(frames).tolist()
    feats = torch.randn(2, 16, 40)
    fmask = (torch.arange(40)[None] < frames[:, None]).long()
    grid = torch.tensor([[1, 4, 4]])
    pix = torch.randn(16, 3 * 2 * 4 * 4)
    # every multimodal span sits between its begin / end markers, as the chat template writes it
    txt = lambda n: torch.randint(0, 180, (n,)).tolist()                                   # noqa: E731
    seq = (txt(2) + [193] + [190] * n_audio[0] + [196] + txt(3) + [194] + [191] * 4 + [195] + txt(2)
           + [193] + [190] * n_audio[1] + [196] + txt(4))
    ids = torch.tensor([seq])
    kw = dict(input_ids=ids, pixel_values=pix, image_grid_thw=grid, input_features=feats, feature_attention_mask=fmask)
    with torch.no_grad():
        want = hf(attention_mask=torch.ones_like(ids), **kw).logits
        got = m(**kw).logits
        torch.testing.assert_close(got, want, atol=4e-4, rtol=4e-4)
        n = ids.shape[1]
        cache = m.init_cache(1, n + 2)
        m(past_key_values=cache, **{**kw, "input_ids": ids[:, :n - 2]})
        cache.advance(n - 2)
        nxt = m(input_ids=ids[:, n - 2:], past_key_values=cache).logits
        torch.testing.assert_close(nxt, want[:, n - 2:], atol=4e-4, rtol=4e-4)
    m.train()
    _, met = m.compute_loss(labels=ids, **kw)
    met.loss.backward()
    assert torch.isfinite(met.loss) and m.audio_tower.conv2d1.weight.grad.abs().sum() > 0
    # names: the thinker's own, and with the "thinker." prefix of the full checkpoint
    ref = hf.state_dict()
    back = _adapt_to_hf_module_names(internal_to_hf(m), ref)
    assert set(back) == set(ref)
    assert all(torch.equal(back[k], ref[k]) for k in ref)
    full = Qwen3OmniMoeForConditionalGeneration(Qwen3OmniMoeConfig(thinker_config=m.config.to_dict()),
                                                dtype=torch.float32)
    full.load_state_dict(hf_to_internal(full, {"thinker." + k: v for k, v in ref.items()}))
    assert all(k.startswith("thinker.") for k in internal_to_hf(full))
