"""Training loop machinery shared by every trainer.

Same responsibilities as easydel/trainers/base_trainer.py:163-5644 and
trainer/trainer.py:57-871: resume from the latest checkpoint, build the data loaders, create
optimizer and state, run epochs of optimizer steps with gradient accumulation, report metrics,
save ``run-<step>`` checkpoints (with ``save_total_limit`` cleanup), evaluate, stop on a time limit
or a break request and return a ``TrainerOutput``.

What differs from the reference is the execution model: a step is not one traced program; it is a
host loop of micro-batches whose backward kernels accumulate into flat fp32 gradient buffers,
followed by the fused optimizer launches of :meth:`EasyDeLState.apply_gradients`. Subclasses
override :meth:`compute_step_loss` (one micro-batch -> ``LossMetrics``) and, when they need it,
:meth:`_preprocess_batch_input` (e.g. RL trainers generate completions there).
"""

from __future__ import annotations

import glob
import json
import math
import os
import re
import shutil
import time
import typing as tp
from dataclasses import dataclass, field

import torch

from ..infra.base_state import EasyDeLState
from ..infra.errors import EasyDeLBreakRequest, EasyDeLPreemptionSignal, EasyDeLTimerError
from ..infra.loss_utils import LossConfig, LossMetrics
from .metrics import MetricsLogger, StepMetrics, create_progress_bar
from .training_configurations import TrainingArguments


@dataclass
class TrainerOutput:
    state: EasyDeLState
    mesh: tp.Any = None
    last_save_file_name: str | None = None
    checkpoint_path: str | None = None
    metrics_history: list = field(default_factory=list)
    interrupted: bool = False


def find_latest_checkpoint(root: str) -> str | None:
    """Newest ``run-<step>`` directory under ``root`` that carries a complete state (metadata written last)."""
    best, best_step = None, -1
    for d in glob.glob(os.path.join(root, "run-*")):
        m = re.search(r"run-(\d+)$", d)
        if not m or not os.path.exists(os.path.join(d, "metadata.json")):
            continue
        if int(m.group(1)) > best_step:
            best, best_step = d, int(m.group(1))
    return best


def _to_device(batch: dict, device, non_blocking: bool = True) -> dict:
    out = {}
    for k, v in batch.items():
        if isinstance(v, torch.Tensor):
            out[k] = v.to(device, non_blocking=non_blocking)
        else:
            out[k] = v
    return out


class BaseTrainer:
    trainer_type = "base"
    arguments_class = TrainingArguments

    def __init__(self, arguments: TrainingArguments | None = None, model=None, model_state: EasyDeLState | None = None,
                 dataset_train=None, dataset_eval=None, data_collator: tp.Callable | None = None,
                 processing_class=None, tokenizer=None, finetune: bool = True, **kwargs):
        if arguments is None:
            arguments = self.arguments_class()
        self.arguments = arguments
        if model is None and model_state is None:
            raise ValueError("pass either `model` or `model_state`")
        self.model = model if model is not None else model_state.model
        self.model_state = model_state
        self.dataset_train, self.dataset_eval = dataset_train, dataset_eval
        self.data_collator = data_collator
        self.processing_class = processing_class if processing_class is not None else tokenizer
        self.finetune = finetune
        self.mesh = getattr(self.model.config, "mesh", None)
        self.device = self.model.device
        self._hooks: dict[str, list[tp.Callable]] = {"on_step_start": [], "on_step_end": [],
                                                     "on_generation_preview": [], "on_benchmark": []}
        self.last_previews: list[str] = []
        self.last_benchmarks: dict = {}
        self._break_requested = False
        self._resumed_from: str | None = None
        self.loss_config = arguments.loss_config or LossConfig()
        if arguments.lmhead_chunksize is not None:
            self.model.config.lmhead_chunksize = arguments.lmhead_chunksize
        self._dp_world, self._dp_rank = self._data_parallel_layout()
        self.initialize_trainer_utils()

    # ------------------------------------------------------------------ setup
    def _data_parallel_layout(self) -> tuple[int, int]:
        mesh = self.mesh
        if mesh is None or not mesh.is_distributed:
            return 1, 0
        return mesh.axis_size(("dp", "fsdp")), mesh.axis_index(("dp", "fsdp"))

    def initialize_trainer_utils(self) -> None:
        a = self.arguments
        self.local_batch_size = max(1, a.total_batch_size // self._dp_world)
        if a.total_batch_size % self._dp_world:
            raise ValueError(f"total_batch_size {a.total_batch_size} not divisible by data-parallel size "
                             f"{self._dp_world}")
        if self.local_batch_size % a.gradient_accumulation_steps:
            raise ValueError(f"per-rank batch {self.local_batch_size} not divisible by gradient_accumulation_steps "
                             f"{a.gradient_accumulation_steps}")
        self.micro_batch_size = self.local_batch_size // a.gradient_accumulation_steps
        self._configure_dataloaders()
        self._configure_state()
        fpt = 0.0
        try:
            fpt = self.model.flops_per_token(sequence_length=a.max_length, include_loss=True)
        except Exception:
            fpt = 0.0
        self.step_metrics = StepMetrics(a, flops_per_token=fpt, world_size=max(1, self._dp_world))
        run_dir = a.get_path() if (a.save_directory and a.can_log_metrics and not a.performance_mode) else None
        self.logger = MetricsLogger(a, run_dir if a.report_metrics and run_dir else None)

    # data ------------------------------------------------------------------
    def _configure_dataloaders(self) -> None:
        a = self.arguments
        self.dataloader_train = self._make_loader(self.dataset_train, self.local_batch_size, a.shuffle_train_dataset,
                                                  a.shuffle_seed_train) if self.dataset_train is not None else None
        self.dataloader_eval = self._make_loader(self.dataset_eval, a.eval_batch_size or self.local_batch_size, False,
                                                 0) if self.dataset_eval is not None else None
        n = self._loader_len(self.dataloader_train)
        if a.max_training_steps is not None:
            self.max_training_steps = a.max_training_steps
            self.steps_per_epoch = n or a.per_epoch_training_steps or a.max_training_steps
        elif n is not None:
            self.steps_per_epoch = a.per_epoch_training_steps or n
            self.max_training_steps = self.steps_per_epoch * a.num_train_epochs
        elif a.per_epoch_training_steps:
            self.steps_per_epoch = a.per_epoch_training_steps
            self.max_training_steps = self.steps_per_epoch * a.num_train_epochs
        else:
            raise ValueError("dataset has no length: set max_training_steps or per_epoch_training_steps")
        a.max_training_steps = self.max_training_steps
        a._setup_optimizer()

    @staticmethod
    def _loader_len(loader) -> int | None:
        try:
            return len(loader)
        except TypeError:
            return None

    def create_collect_function(self, max_sequence_length: int | None = None, truncation_mode: str = "keep_end"):
        """Default collator: stacks equal-length examples, pads ragged ones on the right."""
        from .utils import default_collate

        pad_id = getattr(self.processing_class, "pad_token_id", None) or 0
        return lambda feats: default_collate(feats, pad_token_id=pad_id, max_length=max_sequence_length,
                                             truncation_mode=truncation_mode)

    def _make_loader(self, dataset, batch_size: int, shuffle: bool, seed: int):
        from ..data.loader import build_loader

        collate = self.data_collator or self.create_collect_function(self.arguments.max_length,
                                                                     self.arguments.truncation_mode)
        return build_loader(dataset, batch_size=batch_size, shuffle=shuffle, seed=seed, collate_fn=collate,
                            rank=self._dp_rank, world_size=self._dp_world,
                            num_workers=self.arguments.dataloader_num_workers or 0,
                            pin_memory=bool(self.arguments.dataloader_pin_memory) and torch.cuda.is_available(),
                            drop_last=True)

    # state -----------------------------------------------------------------
    def _configure_state(self) -> None:
        a = self.arguments
        self.tx, self.scheduler = a.get_optimizer_and_scheduler(self.max_training_steps)
        if a.frozen_parameters:
            rx = re.compile(a.frozen_parameters)
            for n, p in self.model.named_parameters():
                if rx.search(n):
                    p.requires_grad_(False)
        resumed = None
        if a.resume_if_possible and a.save_directory:
            latest = find_latest_checkpoint(a.get_path())
            if latest is not None:
                resumed = latest
        if self.model_state is None:
            self.model_state = EasyDeLState.create(model=self.model)
        if resumed is not None:
            from ..io.checkpoint import load_state_into

            load_state_into(self.model_state, resumed, tx=self.tx, load_optimizer=a.save_optimizer_state)
            self._resumed_from = resumed
        if self.model_state.flat is None and a.init_tx:
            self.model_state.init_tx(self.tx)
        elif self.model_state.tx is None:
            self.model_state.tx = self.tx
        if a.step_start_point is not None and (a.force_step_start_point or resumed is None):
            self.model_state.step = a.step_start_point

    # ------------------------------------------------------------------ hooks
    def register_hook(self, name: str, fn: tp.Callable) -> None:
        self._hooks[name].append(fn)

    def request_break(self) -> None:
        self._break_requested = True

    # ------------------------------------------------------------------ per-trainer pieces
    def _preprocess_batch_input(self, state: EasyDeLState, batch: dict, is_train: bool) -> tuple[dict, dict]:
        """Hook run on the host before a step (RL trainers roll out here). Returns (batch, extra metrics)."""
        return batch, {}

    def compute_step_loss(self, model, batch: dict, loss_scale: float, is_train: bool) -> LossMetrics:
        """One micro-batch forward; must return ``LossMetrics`` whose ``loss`` is ready for ``backward``."""
        labels = batch.get("labels")
        call = {k: v for k, v in batch.items() if k != "labels"}
        _, metrics = model.compute_loss(labels=labels, loss_config=self.loss_config, loss_scale=loss_scale, **call)
        return metrics

    def _split_micro(self, batch: dict, n: int) -> list[dict]:
        if n == 1:
            return [batch]
        outs = [dict() for _ in range(n)]
        for k, v in batch.items():
            if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape[0] % n == 0:
                for i, c in enumerate(v.chunk(n, dim=0)):
                    outs[i][k] = c
            else:
                for o in outs:
                    o[k] = v
        return outs

    # ------------------------------------------------------------------ one optimizer step
    def training_step(self, batch: dict) -> tuple[torch.Tensor, torch.Tensor, dict]:
        """Runs one optimizer step on a (device) batch. Returns (loss, grad_norm, auxiliary metric tensors)."""
        a = self.arguments
        model, state = self.model, self.model_state
        model.train()
        accum = a.gradient_accumulation_steps
        total = None
        aux: dict[str, torch.Tensor] = {}
        for mb in self._split_micro(batch, accum):
            m = self.compute_step_loss(model, mb, 1.0 / accum, True)
            m.loss.backward()
            d = m.loss.detach()
            total = d if total is None else total + d
            for k in ("accuracy", "weight_sum"):
                v = getattr(m, k)
                if isinstance(v, torch.Tensor):
                    v = v.detach() / (accum if k == "accuracy" else 1)
                    aux[k] = v if k not in aux else aux[k] + v
            for k, v in (m.other_metrics or {}).items():
                if isinstance(v, torch.Tensor):
                    aux[k] = v.detach() / accum if k not in aux else aux[k] + v.detach() / accum
        grad_norm = state.apply_gradients()
        return total, grad_norm, aux

    @torch.no_grad()
    def evaluation_step(self, batch: dict) -> LossMetrics:
        self.model.eval()
        return self.compute_step_loss(self.model, batch, 1.0, False)

    # ------------------------------------------------------------------ loops
    def train(self) -> TrainerOutput:
        a = self.arguments
        state = self.model_state
        start_step = state.step
        t_begin = time.time()
        pbar = create_progress_bar(a.progress_bar_type, self.max_training_steps, "train",
                                   disabled=not a.can_log_metrics or a.performance_mode and a.progress_bar_type != "json")
        pbar.update(start_step)
        interrupted = False
        last_saved = None
        restore_signals = self._install_preemption_handlers()
        try:
            epoch = start_step // max(1, self.steps_per_epoch)
            while state.step < self.max_training_steps:
                it = self._epoch_iterator(epoch, skip=state.step - epoch * self.steps_per_epoch)
                ran = False
                for batch in it:
                    ran = True
                    if state.step >= self.max_training_steps:
                        break
                    self._run_one_step(batch, epoch, pbar)
                    if a.save_steps and state.step % a.save_steps == 0:
                        last_saved = self._save_checkpoint(state.step)
                    if a.evaluation_steps and self.dataloader_eval is not None and \
                            state.step % a.evaluation_steps == 0:
                        self.eval()
                    if a.generation_interval and a.generation_prompts and state.step % a.generation_interval == 0:
                        self.generate_previews(state.step)
                    if a.benchmark_interval and state.step % a.benchmark_interval == 0:
                        self.run_benchmarks(state.step)
                    limit = a.training_time_seconds
                    if limit is not None and time.time() - t_begin > limit:
                        raise EasyDeLTimerError("training_time_limit reached")
                    if self._preempt_signal is not None:
                        # a preemption notice (SIGTERM from the scheduler, or a signal named in the arguments):
                        # the state of the step that just finished is written before the process is taken away
                        # (easydel/trainers/base_trainer.py:5477-5522)
                        if a.save_tpu_preemption_checkpoints and a.save_directory:
                            last_saved = self._save_checkpoint(state.step)
                        raise EasyDeLPreemptionSignal(f"signal {self._preempt_signal}")
                    if self._break_requested:
                        raise EasyDeLBreakRequest("break requested")
                if not ran:
                    break
                epoch += 1
        except (EasyDeLTimerError, EasyDeLBreakRequest, EasyDeLPreemptionSignal, KeyboardInterrupt) as e:
            interrupted = True
            if a.verbose and a.is_process_zero:
                print(f"[trainer] stopping early at step {state.step}: {type(e).__name__}: {e}")
        finally:
            restore_signals()
            pbar.close()
        if a.do_last_save and a.save_directory and (last_saved is None or not last_saved.endswith(f"run-{state.step}")):
            last_saved = self._save_checkpoint(state.step)
        if a.do_eval and self.dataloader_eval is not None and not interrupted:
            self.eval()
        self.logger.close()
        return TrainerOutput(state=state, mesh=self.mesh, last_save_file_name=last_saved, checkpoint_path=last_saved,
                             metrics_history=self.logger.history, interrupted=interrupted)

    # ------------------------------------------------------------------ preemption, previews, benchmarks
    _preempt_signal = None

    def _install_preemption_handlers(self):
        """SIGTERM (what cluster schedulers send before they take a node away) and SIGUSR1 set a flag that the loop
        reads at the next step boundary. Returns a function that puts the previous handlers back. Only the main
        thread can install handlers; elsewhere this is a no-op."""
        import signal
        import threading

        self._preempt_signal = None
        if threading.current_thread() is not threading.main_thread():
            return lambda: None
        previous = {}

        def on_signal(signum, _frame):
            self._preempt_signal = signal.Signals(signum).name

        for name in getattr(self.arguments, "preemption_signals", None) or ("SIGTERM", "SIGUSR1"):
            sig = getattr(signal, name, None)
            if sig is None:
                continue
            try:
                previous[sig] = signal.signal(sig, on_signal)
            except (ValueError, OSError):
                pass

        def restore():
            for sig, h in previous.items():
                try:
                    signal.signal(sig, h)
                except (ValueError, OSError):
                    pass

        return restore

    @torch.no_grad()
    def generate_previews(self, step: int) -> list[str]:
        """Greedy / sampled continuations of ``arguments.generation_prompts`` from the model being trained, logged
        with the step (the reference's training-time generation previews,
        easydel/trainers/base_trainer.py ``maybe_generate``)."""
        a = self.arguments
        tok = self.processing_class
        if tok is None or not a.generation_prompts:
            return []
        was_training = self.model.training
        self.model.eval()
        texts = []
        try:
            for prompt in a.generation_prompts:
                ids = tok(prompt, return_tensors="pt")["input_ids"] if isinstance(prompt, str) else \
                    torch.tensor([list(prompt)])
                kw = {}
                if a.generation_do_sample:
                    kw.update(do_sample=True, temperature=a.generation_temperature or 1.0,
                              top_p=a.generation_top_p or 1.0, top_k=a.generation_top_k or 0,
                              seed=a.generation_seed)
                out = self.model.generate(ids.to(self.device), max_new_tokens=a.generation_max_new_tokens or 32, **kw)
                new = out.sequences[0, ids.shape[1]:].tolist()
                texts.append(tok.decode(new, skip_special_tokens=True) if hasattr(tok, "decode") else str(new))
        finally:
            self.model.train(was_training)
        self.last_previews = texts
        if a.can_log_metrics and hasattr(self.logger, "log_text"):
            self.logger.log_text("generation_preview", texts, step)
        for fn in self._hooks["on_generation_preview"]:
            fn(self, step, texts)
        return texts

    def run_benchmarks(self, step: int) -> dict:
        """lm-eval tasks named in ``arguments.benchmark_tasks`` through the eSurge adapter, when ``lm_eval`` is
        installed (easydel/infra/elarge/benchmarking.py:40-615 drives the same harness); otherwise the
        ``on_benchmark`` hooks alone run."""
        a = self.arguments
        results: dict = {}
        tasks = getattr(a, "benchmark_tasks", None)
        if tasks:
            try:
                import lm_eval  # noqa: F401

                from ..inference.esurge import eSurge
                from ..inference.evaluations.esurge_eval import eSurgeLMEvalAdapter, run_lm_eval

                was_training = self.model.training
                self.model.eval()
                eng = eSurge(self.model, tokenizer=self.processing_class, max_model_len=a.max_length or 2048,
                             max_num_seqs=a.esurge_max_num_seqs or 16,
                             hbm_utilization=a.esurge_hbm_utilization or 0.3)
                try:
                    results = run_lm_eval(eSurgeLMEvalAdapter(eng, self.processing_class), tasks,
                                          limit=getattr(a, "benchmark_limit", None))
                finally:
                    eng.close()
                    self.model.train(was_training)
            except ImportError:
                if a.verbose and a.is_process_zero:
                    print("[trainer] lm_eval is not installed: benchmark tasks skipped")
        for fn in self._hooks["on_benchmark"]:
            out = fn(self, step)
            if isinstance(out, dict):
                results.update(out)
        if results and a.can_log_metrics:
            flat = {f"benchmark/{k}": v for k, v in results.items() if isinstance(v, (int, float))}
            if flat:
                self.logger.log(flat, step)
        self.last_benchmarks = results
        return results

    def _epoch_iterator(self, epoch: int, skip: int = 0):
        loader = self.dataloader_train
        if hasattr(loader, "set_epoch"):
            loader.set_epoch(epoch)
        it = iter(loader)
        # fast-forward after a resume inside an epoch (easydel/trainers/base_trainer.py:5442)
        for _ in range(max(0, skip)):
            try:
                next(it)
            except StopIteration:
                return iter(())
        return it

    def _run_one_step(self, batch: dict, epoch: int, pbar) -> None:
        a = self.arguments
        state = self.model_state
        for fn in self._hooks["on_step_start"]:
            fn(self, state.step)
        self.step_metrics.start_step()
        batch, extra = self._preprocess_batch_input(state, batch, True)
        if a.ids_to_pop_from_dataset:
            for k in a.ids_to_pop_from_dataset:
                batch.pop(k, None)
        from ..utils.helpers import nvtx_range

        with nvtx_range(f"train_step_{state.step + 1}"):
            dev_batch = _to_device(batch, self.device)
            loss, grad_norm, aux = self.training_step(dev_batch)
        step = state.step
        need_report = (step % max(1, a.report_steps) == 0) or step == self.max_training_steps or \
            a.progress_bar_type == "json"
        if need_report or not a.performance_mode:
            # one device->host read per step: the loss (plus whatever is reported with it)
            lm = LossMetrics(loss=loss, max_grad_norm=grad_norm if a.log_grad_norms else None,
                             accuracy=aux.get("accuracy"), weight_sum=aux.get("weight_sum"),
                             other_metrics={k: v for k, v in aux.items() if k not in ("accuracy", "weight_sum")}
                             or None)
            ids = dev_batch.get("input_ids")
            bsz, seq = (ids.shape[0], ids.shape[1]) if isinstance(ids, torch.Tensor) and ids.dim() == 2 else (
                self.local_batch_size, a.max_length or 0)
            metrics = self.step_metrics.calculate(lm, step, epoch, bsz * self._dp_world, seq,
                                                  state.tx.lr_at(step - 1))
            metrics.update(extra)
            if self.device.type == "cuda":
                # The loss read-back above synchronised the stream: a kernel whose bounded wait ran out has written
                # its code by now. Stop here rather than train on the uninitialised output it left behind.
                from ..ops import _lib

                _lib.check_status(self.device)
            if not math.isfinite(metrics["train/loss"]) and self.loss_config.break_on_nan:
                self._break_requested = True
            for w in a.watchers:
                if w.should_log(step):
                    metrics.update(w.collect(self.model))
            self.last_metrics = metrics
            if a.can_log_metrics:
                self.logger.log(metrics, step)
                pbar.set_postfix(**{k: v for k, v in metrics.items()
                                    if k.split("/")[-1] in ("loss", "learning_rate", "tokens_per_second",
                                                            "max_grad_norm", "accuracy")})
        pbar.update(1)
        for fn in self._hooks["on_step_end"]:
            fn(self, state.step)

    @torch.no_grad()
    def eval(self) -> dict[str, float]:
        if self.dataloader_eval is None:
            return {}
        a = self.arguments
        tot, n = 0.0, 0
        acc = 0.0
        t0 = time.perf_counter()
        for i, batch in enumerate(self.dataloader_eval):
            if a.max_evaluation_steps is not None and i >= a.max_evaluation_steps:
                break
            m = self.evaluation_step(_to_device(batch, self.device))
            tot += float(m.loss)
            if m.accuracy is not None:
                acc += float(m.accuracy)
            n += 1
        self.model.train()
        if n == 0:
            return {}
        out = {"eval/loss": tot / n, "eval/perplexity": math.exp(min(tot / n, 30.0)), "eval/accuracy": acc / n,
               "eval/time": time.perf_counter() - t0}
        if a.can_log_metrics:
            self.logger.log(out, self.model_state.step)
        self.last_eval_metrics = out
        return out

    # ------------------------------------------------------------------ checkpoints
    def _save_checkpoint(self, step: int) -> str | None:
        a = self.arguments
        if not a.save_directory:
            return None
        path = a.step_directory(step)
        if self._dp_world > 1:
            import torch.distributed as dist

            dist.barrier()
        self.model_state.save_state(path, save_optimizer=a.save_optimizer_state, step=step)
        if a.is_process_zero:
            a.save_arguments(path)
            self._cleanup_checkpoints()
        if self._dp_world > 1:
            import torch.distributed as dist

            dist.barrier()
        return path

    def _cleanup_checkpoints(self) -> None:
        lim = self.arguments.save_total_limit
        if not lim:
            return
        runs = []
        for d in glob.glob(os.path.join(self.arguments.get_path(), "run-*")):
            m = re.search(r"run-(\d+)$", d)
            if m:
                runs.append((int(m.group(1)), d))
        runs.sort()
        for _, d in runs[:-lim]:
            shutil.rmtree(d, ignore_errors=True)

    def save_pretrained(self, path: str) -> None:
        self.model.save_pretrained(path)


class Trainer(BaseTrainer):
    """The plain causal-LM trainer (registered as ``"base"``)."""

    trainer_type = "base"
