"""Audio front end of the Whisper pipeline: decoding, resampling, log-mel features and long-form chunking
(easydel/inference/vwhisper/utils.py:55-310; the feature maths is the one Whisper checkpoints were trained with).

Everything runs in torch so the STFT and the mel projection happen on the GPU next to the model; no feature
extractor object from another library is needed (one may still be passed to :class:`vWhisperInference`).
"""

from __future__ import annotations

import io
import math
import shutil
import subprocess
import wave

import numpy as np
import torch

SAMPLE_RATE = 16000
N_FFT = 400
HOP = 160


def _hz_to_mel(f):
    """Slaney scale: linear below 1 kHz, logarithmic above."""
    f = np.asarray(f, dtype=np.float64)
    mel = 3.0 * f / 200.0
    log_region = f >= 1000.0
    mel = np.where(log_region, 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) * (27.0 / math.log(6.4)), mel)
    return mel


def _mel_to_hz(m):
    m = np.asarray(m, dtype=np.float64)
    f = 200.0 * m / 3.0
    log_region = m >= 15.0
    return np.where(log_region, 1000.0 * np.exp(math.log(6.4) / 27.0 * (m - 15.0)), f)


def mel_filter_bank(n_mels: int, n_fft: int = N_FFT, sr: int = SAMPLE_RATE) -> torch.Tensor:
    """Triangular, area-normalised (Slaney) mel filters ``[n_mels, n_fft // 2 + 1]``."""
    n_freq = n_fft // 2 + 1
    fft_freqs = np.linspace(0, sr / 2, n_freq)
    mel_pts = _mel_to_hz(np.linspace(_hz_to_mel(0.0), _hz_to_mel(sr / 2), n_mels + 2))
    fdiff = np.diff(mel_pts)
    ramps = mel_pts[:, None] - fft_freqs[None, :]
    lower = -ramps[:-2] / fdiff[:-1, None]
    upper = ramps[2:] / fdiff[1:, None]
    w = np.maximum(0.0, np.minimum(lower, upper))
    w *= (2.0 / (mel_pts[2:n_mels + 2] - mel_pts[:n_mels]))[:, None]
    return torch.from_numpy(w.astype(np.float32))


def log_mel_spectrogram(audio: torch.Tensor, n_mels: int = 80, n_samples: int | None = 30 * SAMPLE_RATE,
                        filters: torch.Tensor | None = None) -> torch.Tensor:
    """``audio`` ``[B, samples]`` or ``[samples]`` at 16 kHz -> ``[B, n_mels, frames]``.

    Pads (or cuts) to ``n_samples`` first; Hann window of 400, hop 160, power spectrum, mel projection, log10 clipped
    to 8 dB below the maximum of each utterance, then ``(x + 4) / 4``.
    """
    squeeze = audio.dim() == 1
    a = audio[None] if squeeze else audio
    a = a.float()
    if n_samples is not None:
        if a.shape[-1] < n_samples:
            a = torch.nn.functional.pad(a, (0, n_samples - a.shape[-1]))
        else:
            a = a[..., :n_samples]
    window = torch.hann_window(N_FFT, periodic=True, device=a.device)
    spec = torch.stft(a, N_FFT, HOP, window=window, center=True, pad_mode="reflect", return_complex=True)
    power = spec[..., :-1].abs() ** 2
    if filters is None:
        filters = mel_filter_bank(n_mels)
    mel = filters.to(a.device) @ power
    logm = torch.clamp(mel, min=1e-10).log10()
    logm = torch.maximum(logm, logm.amax(dim=(-2, -1), keepdim=True) - 8.0)
    out = (logm + 4.0) / 4.0
    return out[0] if squeeze else out


def resample(audio: np.ndarray, sr_in: int, sr_out: int = SAMPLE_RATE) -> np.ndarray:
    """Band-limited resampling by polyphase filtering (``scipy.signal.resample_poly``)."""
    if sr_in == sr_out:
        return audio.astype(np.float32)
    from scipy.signal import resample_poly

    g = math.gcd(int(sr_in), int(sr_out))
    return resample_poly(audio.astype(np.float64), sr_out // g, sr_in // g).astype(np.float32)


def _decode_wav(data: bytes) -> tuple[np.ndarray, int]:
    with wave.open(io.BytesIO(data), "rb") as w:
        sr, n, width, ch = w.getframerate(), w.getnframes(), w.getsampwidth(), w.getnchannels()
        raw = w.readframes(n)
    if width == 2:
        x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
    elif width == 4:
        x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
    elif width == 1:
        x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    else:
        raise ValueError(f"unsupported WAV sample width {width}")
    if ch > 1:
        x = x.reshape(-1, ch).mean(1)
    return x, sr


def decode_audio(data: bytes, sr: int = SAMPLE_RATE) -> np.ndarray:
    """RIFF/WAVE is decoded in process; anything else goes through an ``ffmpeg`` binary when one is installed."""
    if data[:4] == b"RIFF" and data[8:12] == b"WAVE":
        x, sr_in = _decode_wav(data)
        return resample(x, sr_in, sr)
    ff = shutil.which("ffmpeg")
    if ff is None:
        raise RuntimeError("only WAV input can be decoded without an ffmpeg binary on PATH")
    p = subprocess.run([ff, "-i", "pipe:0", "-ac", "1", "-ar", str(sr), "-f", "f32le", "-hide_banner", "-loglevel",
                        "quiet", "pipe:1"], input=data, stdout=subprocess.PIPE, check=True)
    return np.frombuffer(p.stdout, dtype=np.float32).copy()


def load_audio(source, sr: int = SAMPLE_RATE) -> np.ndarray:
    """Path, bytes, array, or ``{"array": ..., "sampling_rate": ...}`` -> mono float32 at ``sr``."""
    if isinstance(source, dict):
        arr = np.asarray(source.get("array", source.get("raw")), dtype=np.float32)
        return resample(arr, int(source.get("sampling_rate", sr)), sr)
    if isinstance(source, (bytes, bytearray)):
        return decode_audio(bytes(source), sr)
    if isinstance(source, str):
        if source.startswith(("http://", "https://")):
            import requests

            return decode_audio(requests.get(source, timeout=60).content, sr)
        with open(source, "rb") as f:
            return decode_audio(f.read(), sr)
    if isinstance(source, torch.Tensor):
        source = source.detach().cpu().numpy()
    arr = np.asarray(source, dtype=np.float32)
    if arr.ndim != 1:
        raise ValueError("audio must be a single-channel 1-D array")
    return arr


def chunk_iter(audio: np.ndarray, chunk_len: int, stride_left: int, stride_right: int):
    """Overlapping windows over a long recording.

    Yields ``(samples, (length, left, right))``: the first window has no left overlap, the last none on the right;
    consecutive windows advance by ``chunk_len - stride_left - stride_right``.
    """
    n = audio.shape[0]
    step = chunk_len - stride_left - stride_right
    if step <= 0:
        raise ValueError("the strides must be shorter than the chunk")
    start = 0
    while True:
        piece = audio[start:start + chunk_len]
        left = 0 if start == 0 else stride_left
        last = start + chunk_len >= n
        right = 0 if last else stride_right
        if piece.shape[0] > left:
            yield piece, (piece.shape[0], left, right)
        if last:
            break
        start += step
