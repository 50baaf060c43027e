"""Converts checkpoints between the Hugging Face layout and the EasyDeL layout (easydel/scripts/convert_hf_to_easydel.py).

    python -m easydel_b200.scripts.convert_hf_to_easydel --source PATH --out DIR [--to easydel|hf] [--dtype bf16]
                                                         [--task causal-language-model] [--quantize nf4]

``--to easydel`` (default) reads ``model.safetensors`` (+ index) or an EasyDeL directory and writes zarr chunks,
``tensorstore_index.json`` and ``config.json``; ``--to hf`` writes ``model.safetensors`` with Hugging Face parameter
names next to the config. Tokenizer files found in the source are copied along. ``--batch FILE`` converts every
``source out`` pair listed in a text file (the reference's ``convert_hf_to_easydel_batch.py``).
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import sys

import torch

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
_TOKENIZER_FILES = ("tokenizer.json", "tokenizer.model", "tokenizer_config.json", "special_tokens_map.json",
                    "vocab.json", "merges.txt", "generation_config.json", "chat_template.jinja")


def convert(source: str, out: str, to: str = "easydel", dtype: str = "bf16", task: str = "causal-language-model",
            quantize: str | None = None, stream: bool = False) -> str:
    from ..infra.factory import TaskType

    if stream:
        # tensor by tensor, never holding the model: for checkpoints larger than host memory
        if to != "easydel" or quantize:
            raise ValueError("--stream converts Hugging Face safetensors to the EasyDeL layout, without quantisation")
        from ..io.streaming_convert import stream_hf_to_easydel

        os.makedirs(out, exist_ok=True)
        stream_hf_to_easydel(source, out, dtype=_DTYPES[dtype], task=task)
        for name in _TOKENIZER_FILES:
            for src in glob.glob(os.path.join(source, name)):
                shutil.copy2(src, os.path.join(out, os.path.basename(src)))
        return out
    from ..modules.auto import auto_modeling as A
    from ..utils.parameters_transformation import internal_to_hf

    cls = A.resolve_model_class(source, TaskType(task))
    model = cls.from_pretrained(source, dtype=_DTYPES[dtype], param_dtype=_DTYPES[dtype], device="cpu")
    if quantize:
        from ..layers.quantization import EasyDeLQuantizationConfig

        model.quantize(EasyDeLQuantizationConfig(quantize))
    os.makedirs(out, exist_ok=True)
    if to == "easydel":
        model.save_pretrained(out)
    elif to == "hf":
        from safetensors.torch import save_file

        sd = {k: v.detach().contiguous().cpu() for k, v in internal_to_hf(model).items()}
        save_file(sd, os.path.join(out, "model.safetensors"), metadata={"format": "pt"})
        cfg = model.config.to_dict()
        with open(os.path.join(out, "config.json"), "w") as f:
            json.dump(cfg, f, indent=2, default=str)
    else:
        raise ValueError(f"--to must be 'easydel' or 'hf', got {to!r}")
    for name in _TOKENIZER_FILES:
        for src in glob.glob(os.path.join(source, name)):
            shutil.copy2(src, os.path.join(out, os.path.basename(src)))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m easydel_b200.scripts.convert_hf_to_easydel")
    ap.add_argument("--source")
    ap.add_argument("--out")
    ap.add_argument("--to", default="easydel", choices=["easydel", "hf"])
    ap.add_argument("--dtype", default="bf16", choices=sorted(_DTYPES))
    ap.add_argument("--task", default="causal-language-model")
    ap.add_argument("--quantize", default=None)
    ap.add_argument("--batch", default=None, help="text file with one 'source out' pair per line")
    ap.add_argument("--stream", action="store_true",
                    help="convert tensor by tensor without building the model (checkpoints larger than host memory)")
    a = ap.parse_args(argv)
    jobs = []
    if a.batch:
        with open(a.batch) as f:
            jobs = [tuple(line.split()[:2]) for line in f if line.strip() and not line.startswith("#")]
    elif a.source and a.out:
        jobs = [(a.source, a.out)]
    else:
        ap.error("give --source and --out, or --batch")
    failed = 0
    for src, dst in jobs:
        try:
            print("converted", src, "->", convert(src, dst, a.to, a.dtype, a.task, a.quantize, a.stream))
        except Exception as e:  # noqa: BLE001
            failed += 1
            print(f"FAILED {src}: {type(e).__name__}: {e}", file=sys.stderr)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
