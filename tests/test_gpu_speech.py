"""Qwen3-Omni speech stack on the GPU kernels (bf16) against the same modules in fp32 on the CPU."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_talker_and_code2wav_on_the_gpu_match_the_cpu_reference():
    from easydel_b200.modules.qwen3_omni_moe import speech as S

    torch.manual_seed(0)
    pred = dict(vocab_size=64, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=64, num_code_groups=4)
    text = dict(vocab_size=160, hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=64, moe_intermediate_size=128, shared_expert_intermediate_size=128,
                num_experts=4, num_experts_per_tok=2, norm_topk_prob=True,
                rope_parameters={"rope_theta": 10000.0, "rope_type": "default", "mrope_section": [8, 12, 12],
                                 "mrope_interleaved": True})
    cfg = S.Qwen3OmniMoeTalkerConfig(code_predictor_config=pred, text_config=text, num_code_groups=4,
                                     thinker_hidden_size=96, codec_eos_token_id=150, codec_nothink_id=140,
                                     codec_think_bos_id=141, codec_think_eos_id=142, codec_pad_id=143, codec_bos_id=144)
    ref = S.Qwen3OmniMoeTalkerForConditionalGeneration(cfg, dtype=torch.float32).eval()
    gpu = S.Qwen3OmniMoeTalkerForConditionalGeneration(cfg, dtype=torch.bfloat16).eval()
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.cuda()
    emb = torch.randn(1, 40, 256) * 0.5
    pos = torch.stack([torch.arange(40), torch.arange(40) // 2, torch.arange(40) % 5])[:, None]
    with torch.no_grad():
        want_logits, want_h = ref(emb, position_ids=pos)
        got_logits, got_h = gpu(emb.cuda().bfloat16(), position_ids=pos.cuda())
    assert (got_h.float().cpu() - want_h).abs().max() < 0.08 * want_h.abs().max()
    assert (got_logits.float().cpu() - want_logits).abs().max() < 0.08 * want_logits.abs().max()
    codes = gpu.generate_codes(emb.cuda().bfloat16(), torch.randn(1, 2, 256, device="cuda").bfloat16(),
                               torch.zeros(1, 1, 256, device="cuda").bfloat16(), max_new_tokens=4, position_ids=pos.cuda())
    assert codes.shape[:2] == (1, 4) and codes.shape[2] <= 4

    c2w = S.Qwen3OmniMoeCode2WavConfig(codebook_size=32, hidden_size=128, num_attention_heads=2, num_key_value_heads=2,
                                       sliding_window=16, intermediate_size=256, num_hidden_layers=2, num_quantizers=4,
                                       upsample_rates=[2, 2], upsampling_ratios=[2], decoder_dim=64,
                                       layer_scale_initial_scale=0.5)
    dec = S.Qwen3OmniMoeCode2Wav(c2w).eval()
    for n, p in dec.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.05)
    tok = torch.randint(0, 32, (1, 4, 48))
    with torch.no_grad():
        want = dec(tok)
        got = dec.cuda().bfloat16()(tok.cuda()).float().cpu()
    assert got.shape == want.shape
    assert (got - want).abs().max() < 0.1 * want.abs().max() + 1e-3
