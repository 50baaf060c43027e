"""Qwen3-Omni speech stack (talker, code predictor, code-to-waveform decoder) against the Hugging Face classes:
weights are taken from a tiny random transformers model, outputs must agree; the generation loop is checked against a
step-by-step reference built from the same forward passes."""

import pytest
import torch

from easydel_b200.modules.qwen3_omni_moe import speech as S

H = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
HC = pytest.importorskip("transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe")

PRED = dict(vocab_size=64, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, num_code_groups=5)
TEXT = dict(vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, moe_intermediate_size=32, shared_expert_intermediate_size=48,
            num_experts=4, num_experts_per_tok=2, norm_topk_prob=True,
            rope_parameters={"rope_theta": 10000.0, "rope_type": "default", "mrope_section": [2, 3, 3],
                             "mrope_interleaved": True})


CODEC = dict(codec_eos_token_id=90, codec_nothink_id=80, codec_think_bos_id=81, codec_think_eos_id=82, codec_pad_id=83,
             codec_bos_id=84)


def _talkers():
    torch.manual_seed(0)
    hc = HC.Qwen3OmniMoeTalkerConfig(code_predictor_config=dict(PRED), text_config=dict(TEXT), num_code_groups=5,
                                     thinker_hidden_size=48, spatial_merge_size=2, **CODEC)
    hf = H.Qwen3OmniMoeTalkerForConditionalGeneration(hc).eval().float()
    for p in hf.parameters():           # the default init leaves expert tensors empty / zero
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.05)
    cfg = S.Qwen3OmniMoeTalkerConfig(code_predictor_config=dict(PRED), text_config=dict(TEXT), num_code_groups=5,
                                     thinker_hidden_size=48, **CODEC)
    ours = S.Qwen3OmniMoeTalkerForConditionalGeneration(cfg, dtype=torch.float32).eval()
    ours.load_hf_state({"talker." + k: v for k, v in hf.state_dict().items()})
    return hf, ours


def test_code_predictor_matches_hf_and_predicts_greedily():
    hf, ours = _talkers()
    x = torch.randn(2, 4, 64)
    with torch.no_grad():
        for step in (None, 0, 1):
            n = 4 if step is None else step + 2
            a = ours.code_predictor(x[:, :n], step)
            b = hf.code_predictor(inputs_embeds=x[:, :n]).logits
            assert (a - b).abs().max() < 1e-4
        codes, embeds = ours.code_predictor.predict(x[:, :1], x[:, 1:2])
        assert codes.shape == (2, 4) and embeds.shape == (2, 4, 64)
        # the same by hand: grow the sequence one code at a time
        seq = x[:, :2]
        for s in range(4):
            tok = hf.code_predictor(inputs_embeds=seq).logits[:, -1].argmax(-1)
            assert torch.equal(tok, codes[:, s])
            seq = torch.cat([seq, hf.code_predictor.get_input_embeddings()[s](tok)[:, None]], 1)


def test_talker_forward_matches_hf_with_three_stream_positions():
    hf, ours = _talkers()
    torch.manual_seed(1)
    emb = torch.randn(2, 10, 64)
    pos = torch.stack([torch.arange(10), torch.arange(10) // 2, torch.arange(10) % 3])[:, None].expand(3, 2, 10)
    with torch.no_grad():
        logits, hidden = ours(emb, position_ids=pos)
        ref = hf.model(inputs_embeds=emb, position_ids=pos)
        ref_logits = hf.codec_head(ref.last_hidden_state)
    assert (hidden - ref.last_hidden_state).abs().max() < 2e-4
    assert (logits - ref_logits).abs().max() < 2e-4
    th = torch.randn(2, 3, 48)
    with torch.no_grad():
        assert (ours.text_projection(th) - hf.text_projection(th)).abs().max() < 1e-5
        assert (ours.hidden_projection(th) - hf.hidden_projection(th)).abs().max() < 1e-5


def test_talker_generation_loop_against_full_recomputation():
    """Every frame of ``generate_codes`` (cache, code predictor, summed code embeddings + trailing text) must be what a
    full forward over the growing input sequence gives."""
    _, ours = _talkers()
    torch.manual_seed(2)
    prefill, trailing, pad = torch.randn(1, 6, 64), torch.randn(1, 2, 64), torch.randn(1, 1, 64)
    codes = ours.generate_codes(prefill, trailing, pad, max_new_tokens=5)
    assert codes.shape[:2] == (1, 5) and 1 <= codes.shape[2] <= 5
    seq = prefill
    with torch.no_grad():
        for t in range(codes.shape[2]):
            logits, hidden = ours(seq)
            tok = logits[:, -1].argmax(-1)
            assert int(tok) == int(codes[0, 0, t])
            first = ours.codec_embedding(tok)[:, None]
            rest, rest_emb = ours.code_predictor.predict(hidden[:, -1:], first)
            assert torch.equal(rest[0], codes[0, 1:, t])
            nxt = first + rest_emb.sum(1, keepdim=True) + (trailing[:, t:t + 1] if t < 2 else pad)
            seq = torch.cat([seq, nxt], 1)


def test_code2wav_matches_hf_and_chunked_decoding():
    torch.manual_seed(0)
    kw = dict(codebook_size=32, hidden_size=64, num_attention_heads=4, num_key_value_heads=4, sliding_window=6,
              intermediate_size=96, num_hidden_layers=2, num_quantizers=3, upsample_rates=[2, 3], upsampling_ratios=[2],
              decoder_dim=32, layer_scale_initial_scale=0.5)
    hf = H.Qwen3OmniMoeCode2Wav(HC.Qwen3OmniMoeCode2WavConfig(**kw)).eval().float()
    for n, p in hf.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.06)
        elif n.endswith(("alpha", "beta")):
            torch.nn.init.normal_(p, std=0.3)
    ours = S.Qwen3OmniMoeCode2Wav(S.Qwen3OmniMoeCode2WavConfig(**kw)).eval()
    ours.load_hf_state({"code2wav." + k: v for k, v in hf.state_dict().items()})
    codes = torch.randint(0, 32, (2, 3, 20))
    with torch.no_grad():
        a, b = ours(codes), hf(codes)
    assert a.shape == b.shape and a.shape[:2] == (2, 1) and a.shape[2] > 200     # 20 frames, x12 minus the trims
    assert 1e-4 < b.abs().max() < 1.0, "the comparison needs an unsaturated waveform"
    assert (a - b).abs().max() < 1e-3 * b.abs().max()
    with torch.no_grad():
        c, d = ours.chunked_decode(codes, chunk_size=8, left_context_size=3), \
            hf.chunked_decode(codes, chunk_size=8, left_context_size=3)
    assert c.shape == d.shape and (c - d).abs().max() < 1e-3 * d.abs().max()


def test_talker_inputs_match_the_hf_hand_over():
    """User turn with a multimodal span and the final assistant turn, against the two helper methods of the
    transformers model (called on a stand-in that carries just the configuration and the talker)."""
    import types

    hf, ours = _talkers()
    torch.manual_seed(3)
    ids = S.SpeechTokenIds(im_start=180, system=181, user=182, assistant=183, tts_pad=184, tts_bos=185, tts_eos=186,
                           audio=190, image=191, video=192)
    # <start> system .. | <start> user t t <image> <image> t | <start> assistant \n r0 r1 r2 r3
    prompt = torch.tensor([[180, 181, 5, 180, 182, 6, 7, 191, 191, 8, 180, 183, 9]])
    seqs = torch.cat([prompt, torch.tensor([[11, 12, 13, 14]])], 1)
    T = seqs.shape[1]
    emb, hid = torch.randn(1, T, 48), torch.randn(1, T, 48)
    table = torch.nn.Embedding(200, 48)
    with torch.no_grad():
        got, got_ids, trailing, pad_e = S.talker_inputs(ours, seqs, prompt, emb, hid, table, ids, speaker_id=77)
        cfg = types.SimpleNamespace(talker_config=hf.config, tts_pad_token_id=184)
        fake = types.SimpleNamespace(config=cfg, talker=hf)
        mm = (seqs == 190) | (seqs == 191) | (seqs == 192)
        user = H.Qwen3OmniMoeForConditionalGeneration._get_talker_user_parts(fake, 3, 10, mm, hid, emb)
        bos_e, eos_e, pad_ref = hf.text_projection(table(torch.tensor([[185, 186, 184]]))).chunk(3, dim=1)
        asst, asst_ids, trail_ref = H.Qwen3OmniMoeForConditionalGeneration._get_talker_assistant_parts(
            fake, 10, T, 77, emb, pad_ref, bos_e, eos_e)
    want = torch.cat([user, asst], 1)
    assert got.shape == want.shape == (1, 7 + 9, 64)
    assert (got - want).abs().max() < 1e-5 and (trailing - trail_ref).abs().max() < 1e-5
    assert (pad_e - pad_ref).abs().max() < 1e-6
    assert got_ids[0, :7].tolist() == seqs[0, 3:10].tolist() and got_ids[0, 7:].tolist() == asst_ids[0].tolist()


def test_speech_generation_end_to_end_on_a_tiny_model():
    """Thinker -> talker -> waveform through ``generate_speech``: shapes, determinism under a seed, and the talker
    tensors kept out of the thinker's checkpoint."""
    from easydel_b200.modules.qwen3_omni_moe import Qwen3OmniMoeConfig, Qwen3OmniMoeForConditionalGeneration

    A = dict(num_mel_bins=16, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=48, d_model=32, n_window=8,
             output_dim=48, n_window_infer=32, downsample_hidden_size=8, max_source_positions=64)
    V = dict(depth=1, hidden_size=32, intermediate_size=48, num_heads=2, patch_size=4, out_hidden_size=48,
             num_position_embeddings=16, deepstack_visual_indexes=[0])
    T = dict(vocab_size=200, hidden_size=48, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=16, moe_intermediate_size=24, num_experts_per_tok=2, num_experts=4,
             rope_parameters=dict(rope_type="default", rope_theta=1e6, mrope_section=[2, 3, 3], mrope_interleaved=True))
    talker = dict(code_predictor_config=dict(PRED, vocab_size=32), text_config=dict(TEXT, vocab_size=1100),
                  num_code_groups=5, thinker_hidden_size=48, codec_eos_token_id=1090, accept_hidden_layer=1,
                  codec_nothink_id=1080, codec_think_bos_id=1081, codec_think_eos_id=1082, codec_pad_id=1083,
                  codec_bos_id=1084, speaker_id={"Ethan": 1085})
    c2w = dict(codebook_size=32, hidden_size=32, num_attention_heads=2, num_key_value_heads=2, sliding_window=6,
               intermediate_size=48, num_hidden_layers=1, num_quantizers=5, upsample_rates=[2, 2], upsampling_ratios=[2],
               decoder_dim=16)
    torch.manual_seed(0)
    cfg = Qwen3OmniMoeConfig(thinker_config=dict(audio_config=A, vision_config=V, text_config=T, audio_token_id=190,
                                                 image_token_id=191, video_token_id=192, audio_start_token_id=193),
                             talker_config=talker, code2wav_config=c2w, enable_audio_output=True,
                             im_start_token_id=180, im_end_token_id=179, tts_pad_token_id=184, tts_bos_token_id=185,
                             tts_eos_token_id=186, system_token_id=181, user_token_id=182, assistant_token_id=183)
    model = Qwen3OmniMoeForConditionalGeneration(cfg, dtype=torch.float32).eval()
    assert model.talker is not None and model.code2wav is not None
    assert not any(k.startswith(("talker.", "code2wav.")) for k in model.state_dict())
    for p in model.talker.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.3)
    prompt = torch.tensor([[180, 181, 5, 180, 182, 6, 7, 8, 180, 183, 9]])
    seqs, wav = model.generate_speech(prompt, speaker="ethan", thinker_max_new_tokens=6, talker_max_new_tokens=7, seed=1)
    assert seqs.shape[0] == 1 and prompt.shape[1] < seqs.shape[1] <= prompt.shape[1] + 6
    assert wav.dim() == 3 and wav.shape[:2] == (1, 1) and wav.abs().max() <= 1.0
    seqs2, wav2 = model.generate_speech(prompt, speaker=1085, thinker_max_new_tokens=6, talker_max_new_tokens=7, seed=1)
    assert torch.equal(seqs, seqs2) and torch.equal(wav, wav2)
    with pytest.raises(ValueError):
        model.generate_speech(prompt, speaker="nobody")
    model.disable_talker()
    with pytest.raises(ValueError):
        model.generate_speech(prompt)
