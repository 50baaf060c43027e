"""``python -m easydel_b200.inference.vwhisper.cli --model PATH [--serve | --audio FILE]``
(easydel/inference/vwhisper/cli.py)."""

from __future__ import annotations

import argparse
import json


def main(argv=None):
    ap = argparse.ArgumentParser(description="Whisper transcription: one file, or an OpenAI-compatible server")
    ap.add_argument("--model", required=True, help="checkpoint directory (Hugging Face or EasyDeL layout)")
    ap.add_argument("--audio", help="audio file to transcribe")
    ap.add_argument("--serve", action="store_true")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--language")
    ap.add_argument("--task", default="transcribe", choices=["transcribe", "translate"])
    ap.add_argument("--timestamps", action="store_true")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    a = ap.parse_args(argv)
    import torch
    from transformers import AutoTokenizer

    from ...modules.whisper import WhisperForConditionalGeneration
    from . import vWhisperInference, vWhisperInferenceConfig
    from .server import run_server

    dtype = getattr(torch, a.dtype)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model = WhisperForConditionalGeneration.from_pretrained(a.model, dtype=dtype, device=dev)
    tok = AutoTokenizer.from_pretrained(a.model)
    inf = vWhisperInference(model, tok, inference_config=vWhisperInferenceConfig(
        batch_size=a.batch_size, language=a.language, task=a.task, return_timestamps=a.timestamps))
    if a.serve:
        run_server(inf, a.host, a.port)
    elif a.audio:
        print(json.dumps(inf.generate(a.audio), ensure_ascii=False))
    else:
        ap.error("give --audio FILE or --serve")


if __name__ == "__main__":
    main()
