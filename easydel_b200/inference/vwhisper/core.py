"""Long-form speech transcription / translation with a Whisper model
(easydel/inference/vwhisper/core.py:75-620, generation.py).

A recording is cut into overlapping 30-second windows, the windows are decoded in batches with
:meth:`WhisperForConditionalGeneration.generate` (features are computed on the model's device), and the windows'
outputs are stitched: with timestamps, segments are placed on the global time axis and those that lie in a window's
overlap margins are dropped in favour of the neighbour that saw them in full; without timestamps, consecutive token
sequences are joined at their best-matching overlap.
"""

from __future__ import annotations

import numpy as np
import torch

from .audio import SAMPLE_RATE, chunk_iter, load_audio, log_mel_spectrogram, mel_filter_bank
from .config import vWhisperInferenceConfig

TIME_PRECISION = 0.02     # seconds per timestamp token


def merge_token_overlap(left: list[int], right: list[int], max_overlap: int | None = None) -> list[int]:
    """Joins two token sequences whose tail / head cover the same audio.

    Picks the overlap length ``n`` whose aligned tokens agree best (matches / n, small bonus for longer overlaps) and
    keeps the left sequence up to the middle of the overlap and the right one after it.
    """
    if not left:
        return list(right)
    if not right:
        return list(left)
    lim = min(len(left), len(right)) if max_overlap is None else min(len(left), len(right), max_overlap)
    best, best_n = 0.0, 0
    la, ra = np.asarray(left), np.asarray(right)
    for n in range(1, lim + 1):
        m = int((la[-n:] == ra[:n]).sum())
        score = m / n + n / 10000.0
        if m > 1 and score > best:
            best, best_n = score, n
    if best_n == 0 or best < 0.5:
        return list(left) + list(right)
    mid = best_n // 2
    return list(left[:len(left) - best_n + mid]) + list(right[mid:])


class vWhisperInference:
    def __init__(self, model, tokenizer=None, processor=None, inference_config: vWhisperInferenceConfig | None = None,
                 dtype: torch.dtype | None = None):
        self.model = model.eval()
        self.tokenizer = tokenizer if tokenizer is not None else getattr(processor, "tokenizer", None)
        self.processor = processor
        self.config = inference_config or vWhisperInferenceConfig()
        self.dtype = dtype or model.dtype
        self.gen_config = self.config.generation_config or getattr(model, "generation_config", None)
        c = model.config
        self.n_mels = c.num_mel_bins
        self.frames = c.max_source_positions * 2
        self.filters = mel_filter_bank(self.n_mels)
        self.device = next(model.parameters()).device

    # ------------------------------------------------------------------ prompt tokens
    def _token_id(self, name: str) -> int | None:
        if self.tokenizer is None:
            return None
        i = self.tokenizer.convert_tokens_to_ids(name)
        unk = getattr(self.tokenizer, "unk_token_id", None)
        return None if i is None or (unk is not None and i == unk) else int(i)

    def _lookup(self, table: str, key: str) -> int | None:
        t = getattr(self.gen_config, table, None) if self.gen_config is not None else None
        if t and key in t:
            return int(t[key])
        return None

    def no_timestamps_id(self) -> int | None:
        v = getattr(self.gen_config, "no_timestamps_token_id", None) if self.gen_config is not None else None
        return int(v) if v is not None else self._token_id("<|notimestamps|>")

    def prompt_ids(self, language: str | None, task: str | None, return_timestamps: bool) -> list[tuple[int, int]]:
        """``[(position, token)]`` forced after the start token: language, task, no-timestamps."""
        forced, pos = [], 1
        if language is not None:
            lang = language.lower().strip()
            tok = lang if lang.startswith("<|") else f"<|{_LANGUAGE_CODES.get(lang, lang)}|>"
            i = self._lookup("lang_to_id", tok)
            i = self._token_id(tok) if i is None else i
            if i is None:
                raise ValueError(f"unknown language {language!r}")
            forced.append((pos, i))
            pos += 1
        if task is not None or language is not None:
            task = task or "transcribe"
            if task not in ("transcribe", "translate"):
                raise ValueError("task must be 'transcribe' or 'translate'")
            i = self._lookup("task_to_id", task)
            i = self._token_id(f"<|{task}|>") if i is None else i
            if i is not None:
                forced.append((pos, i))
                pos += 1
        if not return_timestamps:
            i = self.no_timestamps_id()
            if i is not None:
                forced.append((pos, i))
        return forced

    # ------------------------------------------------------------------ one batch of windows
    def features(self, windows: list[np.ndarray]) -> torch.Tensor:
        n = self.frames * 160
        buf = torch.zeros(len(windows), n, dtype=torch.float32)
        for i, w in enumerate(windows):
            buf[i, : min(n, w.shape[0])] = torch.from_numpy(np.ascontiguousarray(w[:n]))
        buf = buf.pin_memory().to(self.device, non_blocking=True) if self.device.type == "cuda" else buf
        return log_mel_spectrogram(buf, self.n_mels, None, self.filters).to(self.dtype)

    def _decode_batch(self, windows, forced, return_timestamps, max_length):
        feats = self.features(windows)
        ids = self.model.generate(feats, forced_decoder_ids=forced, max_new_tokens=max_length,
                                  return_timestamps=return_timestamps,
                                  no_timestamps_token_id=self.no_timestamps_id())
        return ids.tolist()

    # ------------------------------------------------------------------ public
    def generate(self, audio_input, chunk_length_s: float = 30.0, stride_length_s=None, batch_size: int | None = None,
                 language: str | None = None, task: str | None = None, return_timestamps: bool | None = None):
        cfg = self.config.replace(batch_size=batch_size, language=language, task=task,
                                  return_timestamps=return_timestamps)
        want_ts = bool(cfg.return_timestamps)
        audio = load_audio(audio_input, SAMPLE_RATE)
        chunk_len = int(round(chunk_length_s * SAMPLE_RATE))
        if stride_length_s is None:
            stride_length_s = chunk_length_s / 6
        if isinstance(stride_length_s, (int, float)):
            stride_length_s = [stride_length_s, stride_length_s]
        sl, sr = (int(round(s * SAMPLE_RATE)) for s in stride_length_s)
        forced = self.prompt_ids(cfg.language, cfg.task, want_ts)
        n_prompt = 1 + len(forced)
        pieces = list(chunk_iter(audio, chunk_len, sl, sr))
        bs = max(1, cfg.batch_size or 1)
        outputs: list[tuple[list[int], tuple[int, int, int], int]] = []
        offset = 0
        step = chunk_len - sl - sr
        for b0 in range(0, len(pieces), bs):
            group = pieces[b0:b0 + bs]
            rows = self._decode_batch([p for p, _ in group], forced, want_ts, cfg.max_length)
            for (_, stride), row in zip(group, rows):
                outputs.append((self._strip(row[n_prompt:]), stride, offset))
                offset += step
        if want_ts:
            chunks = self._stitch_timestamps(outputs)
            toks = [t for c in chunks for t in c["tokens"]]
            text = "".join(c["text"] for c in chunks) if self.tokenizer is not None else None
            for c in chunks:
                c.pop("tokens")
            return {"text": text, "tokens": toks, "chunks": chunks}
        toks: list[int] = []
        for row, _, _ in outputs:
            toks = merge_token_overlap(toks, row)
        return {"text": self._text(toks), "tokens": toks}

    __call__ = generate

    # ------------------------------------------------------------------ helpers
    def _strip(self, row):
        c = self.model.config
        out = []
        for t in row:
            if t == c.eos_token_id:
                break
            out.append(t)
        return out

    def _text(self, toks):
        if self.tokenizer is None:
            return None
        return self.tokenizer.decode(toks, skip_special_tokens=True)

    def _stitch_timestamps(self, outputs):
        ts0 = self.no_timestamps_id() + 1
        segs = []
        for row, (length, left, right), offset in outputs:
            t_off = offset / SAMPLE_RATE
            lo, hi = left / SAMPLE_RATE, (length - right) / SAMPLE_RATE
            cur, start = [], None
            for t in row + [None]:
                if t is not None and t < ts0:
                    cur.append(t)
                    continue
                stamp = None if t is None else (t - ts0) * TIME_PRECISION
                if cur:
                    s = 0.0 if start is None else start
                    e = stamp if stamp is not None else length / SAMPLE_RATE
                    mid = 0.5 * (s + e)
                    # a segment belongs to the window whose un-overlapped core contains its midpoint
                    if lo <= mid <= hi or (left == 0 and mid < lo) or (right == 0 and mid > hi):
                        segs.append({"timestamp": (round(t_off + s, 2), round(t_off + e, 2)), "tokens": cur,
                                     "text": self._text(cur)})
                    cur, start = [], None
                else:
                    start = stamp
        segs.sort(key=lambda s: s["timestamp"][0])
        return segs


_LANGUAGE_CODES = {
    "english": "en", "chinese": "zh", "german": "de", "spanish": "es", "russian": "ru", "korean": "ko", "french": "fr",
    "japanese": "ja", "portuguese": "pt", "turkish": "tr", "polish": "pl", "catalan": "ca", "dutch": "nl",
    "arabic": "ar", "swedish": "sv", "italian": "it", "indonesian": "id", "hindi": "hi", "finnish": "fi",
    "vietnamese": "vi", "hebrew": "he", "ukrainian": "uk", "greek": "el", "malay": "ms", "czech": "cs",
    "romanian": "ro", "danish": "da", "hungarian": "hu", "tamil": "ta", "norwegian": "no", "thai": "th", "urdu": "ur",
    "croatian": "hr", "bulgarian": "bg", "lithuanian": "lt", "latin": "la", "maori": "mi", "malayalam": "ml",
    "welsh": "cy", "slovak": "sk", "telugu": "te", "persian": "fa", "latvian": "lv", "bengali": "bn", "serbian": "sr",
    "azerbaijani": "az", "slovenian": "sl", "kannada": "kn", "estonian": "et", "macedonian": "mk", "breton": "br",
    "basque": "eu", "icelandic": "is", "armenian": "hy", "nepali": "ne", "mongolian": "mn", "bosnian": "bs",
    "kazakh": "kk", "albanian": "sq", "swahili": "sw", "galician": "gl", "marathi": "mr", "punjabi": "pa",
    "sinhala": "si", "khmer": "km", "shona": "sn", "yoruba": "yo", "somali": "so", "afrikaans": "af", "occitan": "oc",
    "georgian": "ka", "belarusian": "be", "tajik": "tg", "sindhi": "sd", "gujarati": "gu", "amharic": "am",
    "yiddish": "yi", "lao": "lo", "uzbek": "uz", "faroese": "fo", "haitian creole": "ht", "pashto": "ps",
    "turkmen": "tk", "nynorsk": "nn", "maltese": "mt", "sanskrit": "sa", "luxembourgish": "lb", "myanmar": "my",
    "tibetan": "bo", "tagalog": "tl", "malagasy": "mg", "assamese": "as", "tatar": "tt", "hawaiian": "haw",
    "lingala": "ln", "hausa": "ha", "bashkir": "ba", "javanese": "jw", "sundanese": "su", "cantonese": "yue",
}
