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
