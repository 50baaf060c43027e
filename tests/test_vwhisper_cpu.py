"""Whisper pipeline on CPU: log-mel features against the Hugging Face extractor, chunking, stitching, server."""

import io
import wave

import numpy as np
import torch

from easydel_b200.inference.vwhisper import (chunk_iter, load_audio, log_mel_spectrogram, merge_token_overlap,
                                             vWhisperInference, vWhisperInferenceConfig)
from easydel_b200.modules.whisper import WhisperConfig, WhisperForConditionalGeneration


def _wav_bytes(x, sr):
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(sr)
        w.writeframes((np.clip(x, -1, 1) * 32767).astype("<i2").tobytes())
    return buf.getvalue()


def test_log_mel_matches_hf_feature_extractor():
    from transformers import WhisperFeatureExtractor

    rng = np.random.default_rng(0)
    audio = (rng.standard_normal(16000 * 3) * 0.1).astype(np.float32)
    for n_mels in (80, 128):
        fe = WhisperFeatureExtractor(feature_size=n_mels)
        ref = fe(audio, sampling_rate=16000, return_tensors="pt").input_features[0]
        got = log_mel_spectrogram(torch.from_numpy(audio), n_mels)
        assert got.shape == ref.shape == (n_mels, 3000)
        assert (got - ref).abs().max() < 2e-4


def test_wav_decode_resample_and_chunks():
    t = np.arange(8000) / 8000.0
    x = 0.5 * np.sin(2 * np.pi * 440 * t)
    a = load_audio(_wav_bytes(x, 8000))
    assert a.shape[0] == 16000 and abs(float(np.abs(a).max()) - 0.5) < 0.02
    assert load_audio({"array": x.astype(np.float32), "sampling_rate": 8000}).shape[0] == 16000
    audio = np.arange(100, dtype=np.float32)
    got = list(chunk_iter(audio, 40, 5, 5))
    assert [g[1] for g in got] == [(40, 0, 5), (40, 5, 5), (40, 5, 0)]
    assert got[1][0][0] == 30 and got[2][0][0] == 60
    covered = np.concatenate([p[l:n - r] for p, (n, l, r) in got])
    assert np.array_equal(covered, audio)


def test_merge_token_overlap():
    assert merge_token_overlap([1, 2, 3, 4, 5, 6], [4, 5, 6, 7, 8]) == [1, 2, 3, 4, 5, 6, 7, 8]
    assert merge_token_overlap([1, 2, 3], [9, 8]) == [1, 2, 3, 9, 8]
    assert merge_token_overlap([], [1]) == [1]
    # one token differs inside the overlap: still joined there
    assert merge_token_overlap([1, 2, 3, 4, 5, 6, 7], [3, 4, 9, 6, 7, 8]) == [1, 2, 3, 4, 9, 6, 7, 8]


class _Tok:
    unk_token_id = None

    def convert_tokens_to_ids(self, t):
        return {"<|en|>": 10, "<|transcribe|>": 11, "<|translate|>": 12, "<|notimestamps|>": 63}.get(t)

    def decode(self, ids, skip_special_tokens=True):
        return "".join(f" w{i}" for i in ids if i < 63 and i > 12)


def _tiny():
    torch.manual_seed(0)
    cfg = WhisperConfig(vocab_size=128, d_model=32, encoder_layers=1, decoder_layers=1, encoder_attention_heads=4,
                        decoder_attention_heads=4, encoder_ffn_dim=64, decoder_ffn_dim=64, num_mel_bins=16,
                        max_source_positions=50, max_target_positions=16, pad_token_id=0, bos_token_id=1,
                        eos_token_id=2, decoder_start_token_id=3)
    return WhisperForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()


def test_long_form_pipeline_and_prompt():
    m = _tiny()
    inf = vWhisperInference(m, _Tok(), inference_config=vWhisperInferenceConfig(batch_size=2, max_length=8))
    assert inf.prompt_ids("english", None, False) == [(1, 10), (2, 11), (3, 63)]
    assert inf.prompt_ids("en", "translate", True) == [(1, 10), (2, 12)]
    audio = (np.random.default_rng(0).standard_normal(16000 * 2) * 0.1).astype(np.float32)
    # windows of 1 s (the tiny model holds 100 frames = 1 s), 0.1 s margins -> 3 windows
    out = inf.generate(audio, chunk_length_s=1.0, stride_length_s=0.1, language="en")
    assert isinstance(out["text"], str) and out["tokens"] and all(t < 63 for t in out["tokens"])
    ts = inf.generate(audio, chunk_length_s=1.0, stride_length_s=0.1, language="en", return_timestamps=True)
    assert ts["chunks"], ts
    starts = [c["timestamp"][0] for c in ts["chunks"]]
    assert starts == sorted(starts) and all(c["timestamp"][1] >= c["timestamp"][0] for c in ts["chunks"])


def test_whisper_server_formats():
    from fastapi.testclient import TestClient

    from easydel_b200.inference.vwhisper.server import create_whisper_app

    class _Fake:
        def generate(self, data, language=None, task=None, return_timestamps=False):
            out = {"text": f"{task}:{language}:{len(data) > 0}"}
            if return_timestamps:
                out["chunks"] = [{"timestamp": (0.0, 1.5), "text": " hello"}, {"timestamp": (1.5, 3.25), "text": " you"}]
            return out

    client = TestClient(create_whisper_app(_Fake()))
    wav = _wav_bytes(np.zeros(1600), 16000)
    r = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav, "audio/wav")}, data={"language": "en"})
    assert r.status_code == 200 and r.json()["text"] == "transcribe:en:True" and r.json()["segments"] is None
    r = client.post("/v1/audio/translations", files={"file": ("a.wav", wav, "audio/wav")},
                    data={"response_format": "text"})
    assert r.text == "translate:None:True"
    r = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav, "audio/wav")},
                    data={"response_format": "srt"})
    assert "00:00:01,500 --> 00:00:03,250" in r.text and r.text.startswith("1\n")
    r = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav, "audio/wav")},
                    data={"response_format": "vtt"})
    assert r.text.startswith("WEBVTT") and "00:00:00.000 --> 00:00:01.500" in r.text
    r = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav, "audio/wav")},
                    data={"response_format": "verbose_json"})
    assert r.json()["segments"][1]["end"] == 3.25 and r.json()["duration"] == 3.25
    assert client.post("/v1/audio/transcriptions", files={"file": ("a.wav", b"", "audio/wav")}).status_code == 400
    assert client.get("/health").json()["status"] == "healthy"
