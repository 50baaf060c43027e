"""Step metrics, progress reporting and tensor watchers.

``StepMetrics.calculate`` produces the same keys as easydel/trainers/metrics.py:93-202 (loss,
perplexity, accuracy, learning rate, grad norm, step time, ``throughput`` = batch*seq/exec_time,
TFLOP/s from the analytic FLOP model); progress bars come in tqdm / json / null flavours
(:469-634); ``LogWatcher`` reports statistics of regex-selected tensors (:776-859).
"""

from __future__ import annotations

import json
import math
import re
import sys
import time
import typing as tp
from dataclasses import dataclass, field

import torch


class StepMetrics:
    def __init__(self, arguments, flops_per_token: float = 0.0, world_size: int = 1):
        self.arguments = arguments
        self.flops_per_token = flops_per_token
        self.world_size = world_size
        self.start_time = time.time()
        self.step_start = None

    def start_step(self) -> None:
        self.step_start = time.perf_counter()

    def calculate(self, metrics, current_step: int, epoch: int, batch_size: int, seq_length: int,
                  learning_rate: float, mode: str = "train", execution_time: float | None = None,
                  n_tokens: int | None = None) -> dict[str, float]:
        exec_time = execution_time if execution_time is not None else (time.perf_counter() - (self.step_start or 0))
        vals = metrics.to_float_dict() if hasattr(metrics, "to_float_dict") else dict(metrics)
        tokens = n_tokens if n_tokens is not None else batch_size * seq_length
        loss = vals.get("loss", float("nan"))
        out = {
            f"{mode}/loss": loss,
            f"{mode}/perplexity": math.exp(min(loss, 30.0)) if loss == loss else float("nan"),
            f"{mode}/step_time": exec_time,
            f"{mode}/throughput": tokens / max(exec_time, 1e-9),
            f"{mode}/tokens_per_second": tokens / max(exec_time, 1e-9),
            f"{mode}/step": current_step,
            f"{mode}/epoch": epoch,
            f"{mode}/total_time": time.time() - self.start_time,
            f"{mode}/visited_tokens": tokens * current_step,
        }
        if mode == "train":
            out["train/learning_rate"] = learning_rate
            if self.flops_per_token:
                total_flops = self.flops_per_token * tokens * 3.0  # forward + backward
                out["train/tflops"] = total_flops / max(exec_time, 1e-9) / 1e12
                out["train/tflops_per_device"] = out["train/tflops"] / max(self.world_size, 1)
        for k in ("accuracy", "z_loss", "weight_sum", "max_grad_norm", "mean_grad_norm"):
            if k in vals:
                out[f"{mode}/{k}"] = vals[k]
        for k, v in vals.items():
            if k not in ("loss", "accuracy", "z_loss", "weight_sum", "max_grad_norm", "mean_grad_norm",
                         "learning_rate", "execution_time"):
                out[f"{mode}/{k}"] = v
        return out


# ------------------------------------------------------------------------------- progress bars
class BaseProgressBar:
    def update(self, n: int = 1) -> None: ...
    def set_postfix(self, **kw) -> None: ...
    def reset(self) -> None: ...
    def close(self) -> None: ...


class NullProgressBar(BaseProgressBar):
    pass


class TqdmProgressBar(BaseProgressBar):
    def __init__(self, total: int, desc: str = "", disabled: bool = False):
        from tqdm import tqdm

        self.bar = tqdm(total=total, desc=desc, disable=disabled, dynamic_ncols=True)

    def update(self, n: int = 1) -> None:
        self.bar.update(n)

    def set_postfix(self, **kw) -> None:
        self.bar.set_postfix({k.split("/")[-1]: (f"{v:.4g}" if isinstance(v, float) else v) for k, v in kw.items()})

    def reset(self) -> None:
        self.bar.reset()

    def close(self) -> None:
        self.bar.close()


class JSONProgressBar(BaseProgressBar):
    def __init__(self, total: int, desc: str = "", stream=None):
        self.total, self.desc, self.n = total, desc, 0
        self.stream = stream or sys.stdout
        self.post: dict = {}

    def update(self, n: int = 1) -> None:
        self.n += n
        rec = {"desc": self.desc, "step": self.n, "total": self.total, **self.post}
        self.stream.write(json.dumps(rec, default=float) + "\n")
        self.stream.flush()

    def set_postfix(self, **kw) -> None:
        self.post = kw


def create_progress_bar(kind: str, total: int, desc: str, disabled: bool = False) -> BaseProgressBar:
    if disabled or kind in ("none", None):
        return NullProgressBar()
    if kind == "json":
        return JSONProgressBar(total, desc)
    # "rich" falls back to tqdm rendering: same information, one dependency fewer
    return TqdmProgressBar(total, desc)


# ------------------------------------------------------------------------------- watchers
@dataclass
class LogWatcher:
    """Reports ``mean / std / abs-max / norm`` of parameters whose name matches ``pattern`` every ``interval`` steps."""

    pattern: str = r".*"
    interval: int = 100
    stats: tuple[str, ...] = ("mean", "std", "absmax", "norm")
    prefix: str = "watch"

    def should_log(self, step: int) -> bool:
        return self.interval > 0 and step % self.interval == 0

    @torch.no_grad()
    def collect(self, model) -> dict[str, float]:
        rx = re.compile(self.pattern)
        out = {}
        for n, p in model.named_parameters():
            if not rx.search(n):
                continue
            pf = p.detach().float()
            if "mean" in self.stats:
                out[f"{self.prefix}/{n}/mean"] = pf.mean().item()
            if "std" in self.stats:
                out[f"{self.prefix}/{n}/std"] = pf.std().item() if pf.numel() > 1 else 0.0
            if "absmax" in self.stats:
                out[f"{self.prefix}/{n}/absmax"] = pf.abs().max().item()
            if "norm" in self.stats:
                out[f"{self.prefix}/{n}/norm"] = pf.norm().item()
        return out


@torch.no_grad()
def compute_weight_stats(model, pattern: str = r".*") -> dict[str, float]:
    return LogWatcher(pattern=pattern, interval=1, prefix="weights").collect(model)


class MetricsLogger:
    """Fans metrics out to the progress bar, a JSONL file, TensorBoard and W&B when those are importable."""

    def __init__(self, arguments, run_dir: str | None = None):
        self.arguments = arguments
        self.history: list[dict] = []
        self._jsonl = None
        self._tb = None
        self._wandb = None
        if run_dir and arguments.can_log_metrics:
            import os

            os.makedirs(run_dir, exist_ok=True)
            self._jsonl = open(os.path.join(run_dir, "metrics.jsonl"), "a", encoding="utf-8")
            try:
                from torch.utils.tensorboard import SummaryWriter  # type: ignore

                self._tb = SummaryWriter(os.path.join(run_dir, "tensorboard"))
            except Exception:
                self._tb = None
            if arguments.use_wandb:
                try:
                    import wandb  # type: ignore

                    self._wandb = wandb.init(project=f"EasyDeL-{arguments.model_name}", name=arguments.wandb_name,
                                             entity=arguments.wandb_entity, config=arguments.to_dict(),
                                             mode="offline")
                except Exception:
                    self._wandb = None

    def log(self, metrics: dict, step: int) -> None:
        self.history.append({"step": step, **metrics})
        if self._jsonl is not None:
            self._jsonl.write(json.dumps({"step": step, **metrics}, default=float) + "\n")
            self._jsonl.flush()
        if self._tb is not None:
            for k, v in metrics.items():
                if isinstance(v, (int, float)):
                    self._tb.add_scalar(k, v, step)
        if self._wandb is not None:
            self._wandb.log(metrics, step=step)

    def log_text(self, key: str, texts: list[str], step: int) -> None:
        """Free text (generation previews) beside the scalar metrics."""
        self.history.append({"step": step, key: list(texts)})
        if self._jsonl is not None:
            self._jsonl.write(json.dumps({"step": step, key: list(texts)}) + "\n")
            self._jsonl.flush()
        if self._tb is not None:
            for i, t in enumerate(texts):
                self._tb.add_text(f"{key}/{i}", t, step)

    def close(self) -> None:
        if self._jsonl is not None:
            self._jsonl.close()
        if self._tb is not None:
            self._tb.close()
        if self._wandb is not None:
            self._wandb.finish()
