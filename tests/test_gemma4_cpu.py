"""Gemma-4 text model against Hugging Face: dense with per-layer inputs and borrowed keys / values, and the variant
with value-less global attention plus the parallel expert block; incremental decoding; training step."""

import pytest
import torch
import transformers

from easydel_b200.modules.gemma4 import Gemma4ForCausalLM, Gemma4TextConfig
from easydel_b200.utils.parameters_transformation import hf_to_internal, internal_to_hf

BASE = dict(vocab_size=160, hidden_size=48, intermediate_size=64, num_hidden_layers=6, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=8, max_position_embeddings=256,
            vocab_size_per_layer_input=160, hidden_size_per_layer_input=12,
            layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2)
VARIANTS = {
    "shared_kv_per_layer_inputs": dict(num_kv_shared_layers=3, use_double_wide_mlp=True, final_logit_softcapping=20.0),
    "k_eq_v_moe": dict(attention_k_eq_v=True, num_global_key_value_heads=1, enable_moe_block=True, num_experts=4,
                       top_k_experts=2, moe_intermediate_size=24, hidden_size_per_layer_input=0),
}


def _pair(name):
    kw = dict(BASE, **VARIANTS[name])
    torch.manual_seed(0)
    hf_cfg = transformers.Gemma4TextConfig(**kw)
    hf_cfg._attn_implementation = "eager"
    hf = transformers.Gemma4ForCausalLM(hf_cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1 or "experts" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("layer_scalar"):
                b.fill_(0.9)
    m = Gemma4ForCausalLM(Gemma4TextConfig(**kw), dtype=torch.float32).eval()
    m.load_state_dict(hf_to_internal(m, hf.state_dict()))
    return hf, m


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_matches_hf_and_decodes_incrementally(name):
    hf, m = _pair(name)
    ids = torch.randint(1, 160, (2, 21))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = m(input_ids=ids).logits
        torch.testing.assert_close(got, want, atol=3e-4, rtol=3e-4)
        cache = m.init_cache(2, 32)
        o = m(input_ids=ids[:, :15], past_key_values=cache).logits
        cache.advance(15)
        torch.testing.assert_close(o, want[:, :15], atol=3e-4, rtol=3e-4)
        for t in range(15, 21):
            o = m(input_ids=ids[:, t:t + 1], past_key_values=cache).logits
            cache.advance(1)
            torch.testing.assert_close(o[:, 0], want[:, t], atol=3e-4, rtol=3e-4)
    back = internal_to_hf(m)
    ref = hf.state_dict()
    for k, v in back.items():
        assert torch.equal(ref[k], v), k


def test_borrowing_layers_hold_no_keys_and_model_trains_and_generates():
    _, m = _pair("shared_kv_per_layer_inputs")
    assert not hasattr(m.model.layers[4].self_attn, "k_proj") and hasattr(m.model.layers[2].self_attn, "k_proj")
    assert m.config.kv_donor(3) == 1 and m.config.kv_donor(5) == 2 and m.config.kv_donor(2) is None
    assert sorted(m.init_cache(1, 8).k) == [0, 1, 2]
    assert m.model.layers[4].mlp.gate_proj.weight.shape[0] == 128
    ids = torch.randint(1, 160, (2, 12))
    m.train()
    _, met = m.compute_loss(input_ids=ids, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss) and m.model.embed_tokens_per_layer.weight.grad.abs().sum() > 0
    m.eval()
    out = m.generate(ids[:, :5], max_new_tokens=4)
    assert out.sequences.shape == (2, 9)


def test_multimodal_matches_hf_with_padded_patches():
    IMG = 150
    text = dict(BASE, num_kv_shared_layers=3)
    vis = dict(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2,
               head_dim=16, pooling_kernel_size=2, patch_size=4, position_embedding_size=64)
    torch.manual_seed(0)
    hf_cfg = transformers.Gemma4Config(text_config=dict(text), vision_config=dict(vis), image_token_id=IMG,
                                       video_token_id=151, audio_token_id=152)
    hf_cfg._attn_implementation = "eager"
    hf_cfg.text_config._attn_implementation = "eager"
    hf_cfg.vision_config._attn_implementation = "eager"
    hf = transformers.Gemma4ForConditionalGeneration(hf_cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1 or "position_embedding_table" in n:
                p.add_(torch.randn_like(p) * 0.1)
    from easydel_b200.modules.gemma4 import Gemma4Config, Gemma4ForConditionalGeneration

    m = Gemma4ForConditionalGeneration(Gemma4Config(text_config=dict(text), vision_config=dict(vis),
                                                    image_token_id=IMG, video_token_id=151, audio_token_id=152),
                                       dtype=torch.float32).eval()
    m.load_state_dict(hf_to_internal(m, hf.state_dict()))
    # image 0: 4 x 6 patches; image 1: 4 x 4 patches plus 8 padding patches; pooled 2 x 2 -> 6 and 4 soft tokens
    def grid(w, h, n):
        xy = torch.stack(torch.meshgrid(torch.arange(w), torch.arange(h), indexing="xy"), -1).reshape(-1, 2)
        return torch.cat([xy, -torch.ones(n - xy.shape[0], 2, dtype=torch.long)])
    pos = torch.stack([grid(6, 4, 24), grid(4, 4, 24)])
    pix = torch.rand(2, 24, 48)
    pix[1, 16:] = 0
    ids = torch.randint(1, 140, (1, 24))
    ids[0, 2:8] = IMG
    ids[0, 11:15] = IMG
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pix, image_position_ids=pos).logits
        feats = m.get_image_features(pix, image_position_ids=pos)
        assert feats.shape == (10, 48)
        ref_feats = hf.model.get_image_features(pix, pos, return_dict=True).pooler_output
        torch.testing.assert_close(feats, ref_feats, atol=2e-4, rtol=2e-4)
        got = m(input_ids=ids, pixel_values=pix, image_position_ids=pos).logits
        torch.testing.assert_close(got, want, atol=4e-4, rtol=4e-4)
        cache = m.init_cache(1, 32)
        m(input_ids=ids[:, :20], pixel_values=pix, image_position_ids=pos, past_key_values=cache)
        cache.advance(20)
        nxt = m(input_ids=ids[:, 20:], past_key_values=cache).logits
        torch.testing.assert_close(nxt, want[:, 20:], atol=4e-4, rtol=4e-4)
    m.train()
    _, met = m.compute_loss(input_ids=ids, labels=ids, pixel_values=pix, image_position_ids=pos)
    met.loss.backward()
    assert m.vision_tower.encoder.layers[0].self_attn.q_proj.linear.weight.grad.abs().sum() > 0
    back = internal_to_hf(m)
    ref = hf.state_dict()
    for k, v in back.items():
        assert torch.equal(ref[k], v), k
