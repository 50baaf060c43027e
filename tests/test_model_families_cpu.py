"""Every table-defined family against the Hugging Face implementation of the same ``model_type``.

A tiny random model is built here in fp32, its weights are exported through the Hugging Face name
map into the ``transformers`` model, and the logits of both are compared on random tokens. The
inverse map (Hugging Face -> this framework) is checked by a state-dict round trip.
"""

import pytest
import torch

import easydel_b200.modules as M
from easydel_b200.utils.parameters_transformation import ModelConverter, hf_to_internal, internal_to_hf

_COMMON = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=8,
               num_key_value_heads=4, max_position_embeddings=256)

CASES = {
    "mistral": dict(sliding_window=32, rope_theta=50000.0),
    "qwen2": dict(rope_theta=1e6),
    "qwen3": dict(head_dim=32),
    "seed_oss": dict(head_dim=16),
    "smollm3": dict(no_rope_layer_interval=2, pad_token_id=0),
    "granite": dict(embedding_multiplier=3.0, logits_scaling=2.0, residual_multiplier=0.5, attention_multiplier=0.1),
    "gemma": dict(head_dim=32),
    "gemma2": dict(head_dim=32, sliding_window=32, query_pre_attn_scalar=24),
    "gemma3_text": dict(head_dim=32, sliding_window=32, query_pre_attn_scalar=24, sliding_window_pattern=2),
    "phi3": dict(pad_token_id=0),
    "olmo": dict(clip_qkv=0.5),
    "olmo2": dict(),
    "olmo3": dict(sliding_window=32),
    "cohere": dict(use_qk_norm=True, logit_scale=0.25),
    "stablelm": dict(partial_rotary_factor=0.5, use_qkv_bias=True),
    "starcoder2": dict(sliding_window=32),
    "glm": dict(head_dim=16, pad_token_id=0),
    "glm4": dict(head_dim=16, pad_token_id=0),
    "mixtral": dict(num_local_experts=4, num_experts_per_tok=2),
    "qwen3_moe": dict(head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True),
    "gpt2": dict(_replace=dict(vocab_size=512, n_embd=128, n_layer=3, n_head=8, n_positions=256)),
    "gpt_neox": dict(_replace=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3,
                                   num_attention_heads=8, max_position_embeddings=256, rotary_pct=0.5)),
    "gptj": dict(_replace=dict(vocab_size=512, n_embd=128, n_layer=3, n_head=8, n_positions=256, rotary_dim=8)),
    "opt": dict(_replace=dict(vocab_size=512, hidden_size=128, ffn_dim=256, num_hidden_layers=3,
                              num_attention_heads=8, max_position_embeddings=256)),
    "phi": dict(),
    "falcon": dict(_replace=dict(vocab_size=512, hidden_size=128, num_hidden_layers=3, num_attention_heads=8,
                                 max_position_embeddings=256)),
    "falcon-new": dict(_replace=dict(vocab_size=512, hidden_size=128, num_hidden_layers=3, num_attention_heads=8,
                                     num_kv_heads=2, new_decoder_architecture=True, max_position_embeddings=256,
                                     bias=True), _type="falcon"),
    "falcon-mha": dict(_replace=dict(vocab_size=512, hidden_size=128, num_hidden_layers=3, num_attention_heads=8,
                                     multi_query=False, parallel_attn=False, max_position_embeddings=256),
                       _type="falcon"),
    "cohere2": dict(sliding_window=32, sliding_window_pattern=2, logit_scale=0.25),
    "deepseek_v3": dict(_replace=dict(vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                                      num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=8,
                                      n_shared_experts=1, n_routed_experts=8, kv_lora_rank=32, q_lora_rank=48,
                                      qk_rope_head_dim=16, v_head_dim=24, qk_nope_head_dim=32, n_group=4,
                                      topk_group=2, num_experts_per_tok=3, first_k_dense_replace=1,
                                      max_position_embeddings=256)),
    "deepseek_v2": dict(_replace=dict(vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                                      num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=8,
                                      n_shared_experts=2, n_routed_experts=8, kv_lora_rank=32, q_lora_rank=None,
                                      qk_rope_head_dim=16, v_head_dim=24, qk_nope_head_dim=32,
                                      num_experts_per_tok=3, first_k_dense_replace=1, max_position_embeddings=256)),
    "glm4_moe_lite": dict(_replace=dict(vocab_size=512, hidden_size=128, intermediate_size=256,
                                        moe_intermediate_size=64, num_hidden_layers=3, num_attention_heads=8,
                                        num_key_value_heads=8, n_shared_experts=1, n_routed_experts=8,
                                        kv_lora_rank=32, q_lora_rank=48, qk_rope_head_dim=16, v_head_dim=24,
                                        qk_nope_head_dim=32, num_experts_per_tok=3, first_k_dense_replace=1,
                                        max_position_embeddings=256, pad_token_id=0)),
    "glm_moe_dsa": dict(_replace=dict(vocab_size=512, hidden_size=128, intermediate_size=256,
                                      moe_intermediate_size=64, num_hidden_layers=3, num_attention_heads=8,
                                      num_key_value_heads=8, n_shared_experts=1, n_routed_experts=8, kv_lora_rank=32,
                                      q_lora_rank=48, qk_rope_head_dim=16, v_head_dim=24, qk_nope_head_dim=32,
                                      num_experts_per_tok=3, first_k_dense_replace=1, max_position_embeddings=256,
                                      index_n_heads=4, index_head_dim=32, index_topk=16, pad_token_id=0,
                                      mlp_layer_types=["dense", "sparse", "sparse"])),
    "glm4_moe": dict(_replace=dict(vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                                   num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=16,
                                   n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, use_qk_norm=True,
                                   first_k_dense_replace=1, max_position_embeddings=256, pad_token_id=0)),
    "exaone4": dict(sliding_window=32, sliding_window_pattern=2, head_dim=16),
    "mpt": dict(_replace=dict(d_model=128, n_heads=8, n_layers=3, max_seq_len=256, vocab_size=512)),
    "gpt_oss": dict(head_dim=16, num_local_experts=4, num_experts_per_tok=2, sliding_window=16, intermediate_size=64,
                    rope_scaling={"rope_type": "yarn", "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                  "truncate": False, "original_max_position_embeddings": 64}),
    "qwen3_next": dict(head_dim=16, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8,
                       linear_value_head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24,
                       shared_expert_intermediate_size=48,
                       layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"]),
    "llama4_text": dict(head_dim=16, intermediate_size=48, intermediate_size_mlp=96, num_local_experts=4,
                        num_experts_per_tok=1, attention_chunk_size=32, floor_scale=16, attn_scale=0.3,
                        no_rope_layers=[1, 1, 1, 0], moe_layers=[0, 2, 3],
                        layer_types=["chunked_attention", "chunked_attention", "chunked_attention",
                                     "full_attention"]),
    "phimoe": dict(num_local_experts=4, num_experts_per_tok=2, intermediate_size=96, router_jitter_noise=0.05),
    "qwen3_5_text": dict(head_dim=16, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8,
                         linear_value_head_dim=16,
                         layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"]),
    "qwen3_5_moe_text": dict(head_dim=16, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8,
                             linear_value_head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24,
                             shared_expert_intermediate_size=48,
                             layer_types=["linear_attention", "linear_attention", "linear_attention",
                                          "full_attention"]),
    "falcon_h1": dict(mamba_d_ssm=64, mamba_n_heads=4, mamba_d_head=16, mamba_n_groups=2, mamba_d_state=8,
                      mamba_chunk_size=8, key_multiplier=0.7, attention_in_multiplier=1.3,
                      attention_out_multiplier=0.8, ssm_out_multiplier=0.6, ssm_in_multiplier=1.2,
                      ssm_multipliers=[0.5, 1.5, 0.7, 1.1, 0.9], mlp_multipliers=[0.8, 1.25],
                      embedding_multiplier=2.0, lm_head_multiplier=0.5, mamba_rms_norm=True),
    "minimax": dict(head_dim=16, num_local_experts=4, num_experts_per_tok=2, intermediate_size=96, block_size=16,
                    layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"],
                    full_attn_alpha_factor=1.5, full_attn_beta_factor=0.8, linear_attn_alpha_factor=1.2,
                    linear_attn_beta_factor=0.9, mlp_alpha_factor=1.1, mlp_beta_factor=0.7),
    "qwen2_moe": dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                      shared_expert_intermediate_size=96),
}


def _build(model_type, extra):
    from easydel_b200.infra.factory import TaskType, registry

    extra = dict(extra)
    model_type = extra.pop("_type", model_type)
    base = extra.pop("_replace", None)
    cfg_cls = registry.get_config(model_type)
    cfg = cfg_cls(**({**_COMMON, **extra} if base is None else base))
    reg = registry.get_module_registration(TaskType.CAUSAL_LM, model_type)
    torch.manual_seed(0)
    model = reg.module(cfg, dtype=torch.float32, param_dtype=torch.float32)
    # make every norm scale / bias informative
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)
    return model.eval()


# compared separately: needs explicit causal masks on the transformers side and a length without near-ties
_OWN_TEST = {"glm_moe_dsa"}


@pytest.mark.parametrize("model_type", sorted(set(CASES) - _OWN_TEST))
def test_family_matches_hf(model_type):
    model = _build(model_type, CASES[model_type])
    hf = ModelConverter.easydel_to_huggingface(model, dtype=torch.float32).eval()
    ids = torch.randint(0, 512, (2, 96), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        ours = model(input_ids=ids).logits
        theirs = hf(input_ids=ids).logits
    err = (ours - theirs).abs().max().item()
    assert err < 2e-3 * max(1.0, theirs.abs().max().item()), err
    # Hugging Face names -> internal layout reproduces the original tensors
    back = hf_to_internal(model, hf.state_dict(), strict=True)
    for k, v in model.state_dict().items():
        assert torch.equal(back[k].to(v.dtype), v), k


@pytest.mark.parametrize("model_type", ["qwen3_next", "llama4_text", "gpt_oss", "falcon_h1", "minimax"])
def test_incremental_decoding_matches_full_forward(model_type):
    """Prefill + single-token steps through the dense cache reproduce one full forward: hybrid state for the
    Gated-DeltaNet layers (qwen3_next), block-diagonal attention across a block boundary (llama4), sinks with
    sliding windows (gpt_oss)."""
    torch.manual_seed(0)
    m = _build(model_type, CASES[model_type])
    n, pre = 40, 30
    ids = torch.randint(0, 512, (2, n))
    with torch.no_grad():
        full = m(input_ids=ids).logits
        cache = m.init_cache(2, 48)
        if model_type == "qwen3_next":
            assert set(cache.linear) == {0, 1, 2}
        o = m(input_ids=ids[:, :pre], past_key_values=cache).logits
        cache.advance(pre)
        assert (o - full[:, :pre]).abs().max() < 3e-4
        for t in range(pre, n):
            o = m(input_ids=ids[:, t:t + 1], past_key_values=cache).logits
            cache.advance(1)
            assert (o[:, 0] - full[:, t]).abs().max() < 3e-4, t


def test_glm_moe_dsa_sparse_attention_matches_hf():
    """Top-16 key selection is active (40 tokens). The transformers model runs with eager attention: with its
    default kernel it drops the causal mask whenever the selection mask is present. Longer random sequences contain
    near-ties in the scorer, where the two implementations may legitimately pick different keys."""
    model = _build("glm_moe_dsa", CASES["glm_moe_dsa"])
    hf = ModelConverter.easydel_to_huggingface(model, dtype=torch.float32).eval()
    hf.config._attn_implementation = "eager"
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        ours, theirs = model(input_ids=ids).logits, hf(input_ids=ids).logits
    assert (ours - theirs).abs().max() < 2e-3
    sel = model.model.layers[0].self_attn
    bias = sel._index_bias(torch.randn(1, 40, 128), torch.randn(1, 40, 48), torch.arange(40)[None], None, 40)
    assert int((bias[0, 0, 39] == 0).sum()) == 16 and int((bias[0, 0, 5] == 0).sum()) == 16
    back = hf_to_internal(model, hf.state_dict(), strict=True)
    for k, v in model.state_dict().items():
        assert torch.equal(back[k].to(v.dtype), v), k
    # decoding keeps the scorer's keys in the cache: a step sees all earlier keys
    cache = model.init_cache(2, 48)
    with torch.no_grad():
        model(input_ids=ids[:, :30], past_key_values=cache)
        cache.advance(30)
        model(input_ids=ids[:, 30:31], past_key_values=cache)
    assert cache.index_keys[0].shape[1] == 31
