"""Whisper (speech encoder-decoder) against Hugging Face on CPU: logits, loss, greedy generation, classification."""

import torch
import transformers

from easydel_b200.modules.whisper import (WhisperConfig, WhisperForAudioClassification,
                                          WhisperForConditionalGeneration)
from easydel_b200.utils.parameters_transformation import hf_to_internal, internal_to_hf

KW = dict(vocab_size=128, d_model=32, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
          decoder_attention_heads=4, encoder_ffn_dim=64, decoder_ffn_dim=64, num_mel_bins=16,
          max_source_positions=20, max_target_positions=24, pad_token_id=0, bos_token_id=1, eos_token_id=2,
          decoder_start_token_id=3)


def _pair():
    torch.manual_seed(0)
    m = WhisperForConditionalGeneration(WhisperConfig(**KW), dtype=torch.float32, param_dtype=torch.float32).eval()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)
    hf = transformers.WhisperForConditionalGeneration(transformers.WhisperConfig(**KW)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    return m, hf


def test_whisper_logits_loss_and_roundtrip():
    m, hf = _pair()
    feats = torch.randn(2, 16, 40)
    dec = torch.randint(4, 128, (2, 9))
    with torch.no_grad():
        a = m(input_features=feats, decoder_input_ids=dec).logits
        b = hf(input_features=feats, decoder_input_ids=dec).logits
    assert (a - b).abs().max() < 2e-4
    labels = dec.clone()
    labels[0, -3:] = -100
    la, lb = m(input_features=feats, labels=labels).loss, hf(input_features=feats, labels=labels).loss
    assert abs(float(la) - float(lb)) < 1e-4
    la.backward()
    assert m.model.encoder.conv1.weight.grad.abs().sum() > 0
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_features=feats, labels=labels)
    assert abs(float(met.loss) - float(lb)) < 1e-4


def test_whisper_generate_matches_stepwise_full_forward():
    m, hf = _pair()
    feats = torch.randn(2, 16, 40)
    out = m.generate(feats, max_new_tokens=10, forced_decoder_ids=[(1, 7), (2, 9)], eos_token_id=-1)
    assert out.shape == (2, 11) and (out[:, 1] == 7).all() and (out[:, 2] == 9).all()
    # every generated token is the arg-max of a full (cache-free) forward over its prefix
    with torch.no_grad():
        full = hf(input_features=feats, decoder_input_ids=out[:, :-1]).logits
    for t in range(3, 11):
        assert torch.equal(out[:, t], full[:, t - 1].argmax(-1))


def test_whisper_timestamp_rules_yield_paired_monotonic_stamps():
    m, _ = _pair()
    feats = torch.randn(1, 16, 40)
    no_ts = 63         # tokens 64.. act as timestamps, 2 is EOS
    out = m.generate(feats, max_new_tokens=16, return_timestamps=True, no_timestamps_token_id=no_ts,
                     eos_token_id=2)[0, 1:].tolist()
    assert out[0] >= 64
    stamps = [t for t in out if t >= 64]
    assert stamps == sorted(stamps)
    assert no_ts not in out


def test_whisper_audio_classification_matches_hf():
    kw = dict(KW, use_weighted_layer_sum=True, classifier_proj_size=8, num_labels=3)
    torch.manual_seed(1)
    m = WhisperForAudioClassification(WhisperConfig(**kw), dtype=torch.float32, param_dtype=torch.float32).eval()
    hf = transformers.WhisperForAudioClassification(transformers.WhisperConfig(**kw)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    feats = torch.randn(2, 16, 40)
    with torch.no_grad():
        a, b = m(input_features=feats).logits, hf(input_features=feats).logits
    assert a.shape == (2, 3) and (a - b).abs().max() < 2e-4
