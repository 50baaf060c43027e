"""``eSurge``: the continuous-batching inference engine.

Public behaviour follows easydel/inference/esurge/esurge_engine.py:385-1168 and its mixins:
``generate`` / ``stream`` / ``chat``, ``abort_request``, ``pause`` / ``resume`` / ``terminate``,
``update_model_weights``, metrics summary, a background scheduler thread with an error budget
(``EASURGE_MAX_SCHEDULER_ERRORS``) and a heartbeat. The engine owns: the paged KV cache sized from
free HBM x ``hbm_utilization``, the page pool with prefix caching, the token-budget scheduler and
the model runner.
"""

from __future__ import annotations

import itertools
import os
import threading
import time
import typing as tp
from dataclasses import dataclass, field

import torch

from ...caching.paged import PAGE_SIZE, PagedKVCache
from ..sampling_params import SamplingParams
from .metrics import MetricsCollector
from .kv_manager import KVCacheCoordinator
from .page_pool import PagePool
from .runner import ModelRunner
from .scheduler import EngineRequest, RequestStatus, Scheduler, SchedulerConfig


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    finish_reason: str | None = None
    cumulative_logprob: float | None = None


@dataclass
class RequestOutput:
    request_id: str
    prompt: str | None
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool = False
    delta_text: str = ""
    delta_token_ids: list[int] = field(default_factory=list)
    tokens_per_second: float = 0.0
    num_generated_tokens: int = 0
    time_to_first_token: float | None = None
    processing_time: float = 0.0
    num_cached_tokens: int = 0

    @property
    def accumulated_text(self) -> str:
        return self.outputs[0].text if self.outputs else ""

    def get_text(self) -> str:
        return self.accumulated_text


class IncrementalDetokenizer:
    """Turns a growing token list into text deltas without re-decoding the whole sequence and without
    emitting half of a multi-byte character (the job of the reference's detokenizer worker,
    easydel/workers/esurge/pipeline/worker_main.py:40-374)."""

    def __init__(self, tokenizer, skip_special_tokens: bool = True, window: int = 6):
        self.tok, self.skip, self.window = tokenizer, skip_special_tokens, window
        self.ids: list[int] = []
        self.prefix_offset = 0
        self.read_offset = 0
        self.text = ""

    def push(self, new_ids: tp.Sequence[int]) -> str:
        if self.tok is None:
            return ""
        self.ids.extend(new_ids)
        prefix = self.tok.decode(self.ids[self.prefix_offset:self.read_offset], skip_special_tokens=self.skip)
        full = self.tok.decode(self.ids[self.prefix_offset:], skip_special_tokens=self.skip)
        if full.endswith("�") or len(full) <= len(prefix):
            return ""
        delta = full[len(prefix):]
        self.prefix_offset = max(self.read_offset - self.window, 0)
        self.read_offset = len(self.ids)
        self.text += delta
        return delta


class _Tracked:
    def __init__(self, req: EngineRequest, prompt: str | None, detok: IncrementalDetokenizer):
        self.req, self.prompt, self.detok = req, prompt, detok
        self.event = threading.Event()
        self.lock = threading.Lock()
        self.pending_delta = ""
        self.pending_ids: list[int] = []
        self.start = time.time()
        self.finished = False
        self.finish_reason: str | None = None
        self.emitted_tokens = 0


# Options of the reference engine that steer its ahead-of-time XLA compilation or its process layout; accepted so
# that configurations written for it load, and without effect here.
_COMPILE_ONLY_OPTIONS = frozenset({
    "dtype", "min_input_pad", "min_token_pad", "max_num_seq_buckets", "use_aot_forward", "bind_graphstate_for_aot",
    "auto_shard_model", "compile_runner", "runner_verbose", "sampler_metrics", "data_parallelism_axis",
    "strict_context", "prefer_preserve_prompt", "decode_truncated_prompt", "destroy_pages_on_pause",
    "detokenizer_max_states", "tokenizer_endpoint", "detokenizer_endpoint", "worker_startup_timeout",
    "max_request_outputs", "idle_reset_seconds", "idle_reset_min_interval", "ignore_stop_strings_in_reasoning",
    "resolution_buckets", "vision_cache_capacity_mb"})


class eSurge:
    def __init__(self, model, tokenizer=None, processor=None, max_model_len: int = 8192, max_num_seqs: int = 256,
                 max_num_batched_tokens: int | None = None, hbm_utilization: float = 0.85, page_size: int = PAGE_SIZE,
                 enable_prefix_caching: bool = True, num_pages: int | None = None,
                 long_prefill_token_threshold: int | None = None, scheduling_policy: str = "fcfs",
                 overlap_execution: bool | None = None, async_scheduling: bool | None = None,
                 esurge_name: str | None = None, reserve_tokens: int | None = None,
                 auto_truncate_prompt: bool = True, truncate_mode: str = "left", silent_mode: bool = True,
                 sharding_axis_dims=(1, 1, 1, -1, 1), extra_eos_token_ids: tp.Sequence[int] | None = None,
                 extra_stops: str | tp.Sequence[str] | None = None, auto_cap_new_tokens: bool = True,
                 sampling_params_callback: tp.Callable | None = None, tool_parser: str | None = None,
                 reasoning_parser: str | None = None, kv_quantization=None, **compile_options):
        """``async_scheduling`` / ``overlap_execution`` (either one; default on for CUDA models): step *t+1* is
        scheduled and launched before the tokens of step *t* are read back, so host work overlaps device work.

        ``compile_options`` takes only the reference's ahead-of-time compilation knobs, which have nothing to
        act on here (kernels are launched eagerly or replayed from CUDA graphs); any other name is an error."""
        unknown = set(compile_options) - _COMPILE_ONLY_OPTIONS
        if unknown:
            raise TypeError(f"eSurge got unexpected option(s) {sorted(unknown)}")
        self.model = model.eval() if hasattr(model, "eval") else model
        self.tokenizer = tokenizer if tokenizer is not None else getattr(processor, "tokenizer", processor)
        self.processor = processor
        self._mm = None
        self.max_model_len, self.max_num_seqs = max_model_len, max_num_seqs
        if max_num_batched_tokens is None:
            # the reference's GPU default: min(max(2048, max_num_seqs), max_model_len)
            max_num_batched_tokens = min(max(2048, max_num_seqs), max_model_len)
        self.max_num_batched_tokens = max(max_num_batched_tokens, max_num_seqs)
        self.page_size = page_size
        self.auto_truncate_prompt, self.truncate_mode = auto_truncate_prompt, truncate_mode
        self.reserve_tokens = reserve_tokens if reserve_tokens is not None else 1
        self.name = esurge_name or f"esurge-{id(self) & 0xffff:x}"
        pages_cap = max_num_seqs * ((max_model_len + page_size - 1) // page_size) + 1
        # the page count is settled before anything is allocated: two caches never exist at once
        if kv_quantization is not None:
            # ``kv_quantization``: a ``TurboQuantConfig``; keys and values are stored compressed and attention runs
            # as tensor code over them (no decode graphs)
            from ...caching.turboquant_paged import TurboQuantPagedKVCache

            self.cache = TurboQuantPagedKVCache.init_for_model(getattr(model, "language_model", model),
                                                               kv_quantization, num_pages=num_pages,
                                                               hbm_utilization=hbm_utilization,
                                                               max_pages=pages_cap if num_pages is None else None)
        else:
            self.cache = PagedKVCache.init_for_model(model, num_pages=num_pages, page_size=page_size,
                                                     hbm_utilization=hbm_utilization, max_model_length=max_model_len,
                                                     max_pages=pages_cap if num_pages is None else None,
                                                     max_num_seqs=max_num_seqs,
                                                     max_num_batched_tokens=self.max_num_batched_tokens)
        # hybrids: one recurrent-state row per engine slot (the last row belongs to the padding rows of a batch
        # bucket). A cached prefix has no recurrent state to resume from, so prefix caching is off for them.
        self.cache.add_state_pools(getattr(model, "language_model", model), max_num_seqs + 1)
        if self.cache.linear:
            enable_prefix_caching = False
        # one page pool per cache group (full attention / each sliding window / each chunked-local block size)
        self.kv = KVCacheCoordinator(self.cache.groups, enable_caching=enable_prefix_caching)
        self.pool = self.kv.pool
        self.scheduler = Scheduler(SchedulerConfig(max_num_seqs=max_num_seqs,
                                                   max_num_batched_tokens=self.max_num_batched_tokens,
                                                   max_model_len=max_model_len,
                                                   long_prefill_token_threshold=long_prefill_token_threshold,
                                                   policy=scheduling_policy), self.kv, page_size)
        self.runner = ModelRunner(model, self.cache, max_num_seqs, self.max_num_batched_tokens, max_model_len)
        self.metrics = MetricsCollector()
        self._tracked: dict[str, _Tracked] = {}
        self._free_slots = list(range(max_num_seqs - 1, -1, -1))
        self._ids = itertools.count()
        self._lock = threading.RLock()
        self._work = threading.Condition(self._lock)
        self._thread: threading.Thread | None = None
        self._running = False
        self._paused = False
        self._errors = 0
        self._max_errors = int(os.environ.get("EASURGE_MAX_SCHEDULER_ERRORS", "3"))
        self.last_heartbeat = time.time()
        self.eos_token_id = getattr(model.config, "eos_token_id", None)
        extra_eos = list(extra_eos_token_ids or [])
        if isinstance(self.eos_token_id, (list, tuple)):
            extra_eos = list(self.eos_token_id[1:]) + extra_eos
            self.eos_token_id = self.eos_token_id[0] if self.eos_token_id else None
        self.extra_eos_token_ids = [int(t) for t in extra_eos]
        self.extra_stops = [extra_stops] if isinstance(extra_stops, str) else list(extra_stops or [])
        self.auto_cap_new_tokens = auto_cap_new_tokens
        self.sampling_params_callback = sampling_params_callback
        self.tool_parser, self.reasoning_parser = tool_parser, reasoning_parser
        want_async = async_scheduling if async_scheduling is not None else overlap_execution
        if want_async is None:
            want_async = self.runner.device.type == "cuda"
        self.async_scheduling = bool(want_async)
        self._inflight = None      # (SchedulerOutput, runner handle, launch time) of the step not read back yet

    # ------------------------------------------------------------------ lifecycle
    def initiate(self) -> "eSurge":
        """Starts the background scheduler thread (idempotent)."""
        with self._lock:
            if self._thread is not None and self._thread.is_alive():
                return self
            self._running = True
            self._thread = threading.Thread(target=self._loop, name=f"{self.name}-scheduler", daemon=True)
            self._thread.start()
        return self

    def terminate(self) -> None:
        with self._work:
            self._running = False
            self._work.notify_all()
        if self._thread is not None:
            self._thread.join(timeout=30)
            self._thread = None
        self._drain()

    def _drain(self) -> None:
        """Reads back (and commits) a step that is still in flight."""
        with self._lock:
            prev, self._inflight = self._inflight, None
            if prev is not None:
                self._commit(*prev)

    def close(self) -> None:
        """Stops the scheduler thread, finishes the step in flight and drops the captured CUDA graphs and the
        runner's device buffers, so that the process group can be destroyed and the process can exit."""
        self.terminate()
        self.stop_monitoring()
        self.runner.release()

    def pause(self) -> None:
        with self._work:
            self._paused = True

    def resume(self) -> None:
        with self._work:
            self._paused = False
            self._work.notify_all()

    def start_monitoring(self, prometheus_port: int = 9090, console: bool = False, update_interval: float = 1.0):
        """Starts the Prometheus exporter (and optionally the console monitor) for this engine."""
        from .monitoring import eSurgeMonitoringServer

        if getattr(self, "_monitor", None) is None:
            self._monitor = eSurgeMonitoringServer(self, prometheus_port=prometheus_port, console=console)
            self._monitor.start(update_interval)
        return {"prometheus": f"http://0.0.0.0:{prometheus_port}/metrics"}

    def stop_monitoring(self) -> None:
        mon = getattr(self, "_monitor", None)
        if mon is not None:
            mon.stop()
            self._monitor = None

    def start_profiling(self, output_dir: str = "esurge_profile", record_shapes: bool = False) -> None:
        """Records engine steps with the torch profiler (CPU + CUDA activities) until :meth:`stop_profiling`
        (easydel/inference/esurge/mixins/lifecycle.py:723-815)."""
        if getattr(self, "_profiler", None) is not None:
            raise RuntimeError("profiling is already running")
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._profile_dir = output_dir
        self._profiler = torch.profiler.profile(activities=acts, record_shapes=record_shapes)
        self._profiler.__enter__()

    def stop_profiling(self) -> str | None:
        """Stops the profiler and writes a Chrome trace; returns its path."""
        prof = getattr(self, "_profiler", None)
        if prof is None:
            return None
        prof.__exit__(None, None, None)
        self._profiler = None
        os.makedirs(self._profile_dir, exist_ok=True)
        path = os.path.join(self._profile_dir, f"{self.name}-{int(time.time())}.json")
        prof.export_chrome_trace(path)
        return path

    def update_model_weights(self, model=None, state_dict: dict | None = None) -> None:
        """Swaps in new weights (RL trainers refresh the policy between rollouts). Cached prefixes are dropped."""
        with self._lock:
            if self.scheduler.has_unfinished() or self._inflight is not None:
                raise RuntimeError("cannot update weights while requests are in flight")
            if state_dict is not None:
                self.model.load_state_dict(state_dict, strict=False)
            elif model is not None and model is not self.model:
                self.model.load_state_dict(model.state_dict(), strict=False)
            for m in self.kv.managers:
                m.pool.reset_cache()

    # ------------------------------------------------------------------ requests
    def _tokenize(self, prompt) -> tuple[list[int], str | None]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("string prompts need a tokenizer")
            return list(self.tokenizer(prompt, add_special_tokens=True)["input_ids"]), prompt
        if isinstance(prompt, dict) and "prompt_token_ids" in prompt:
            return list(prompt["prompt_token_ids"]), prompt.get("prompt")
        return [int(t) for t in prompt], None

    @property
    def multimodal(self):
        """The image front end (vision tower runs, feature cache); built on first use for models that have a tower."""
        if self._mm is None and hasattr(self.model, "get_image_features"):
            from .multimodal import MultiModalManager

            self._mm = MultiModalManager(self.model, tokenizer=self.tokenizer, processor=self.processor)
        return self._mm

    def add_request(self, prompt, sampling_params: SamplingParams | None = None, request_id: str | None = None,
                    priority: int = 0, images: tp.Sequence[tp.Any] | None = None,
                    videos: tp.Sequence[tp.Any] | None = None) -> str:
        sp = sampling_params or SamplingParams()
        if self.sampling_params_callback is not None:
            sp = self.sampling_params_callback(sp, {"prompt": prompt, "request_id": request_id}) or sp
        if self.extra_eos_token_ids or self.extra_stops:
            sp = sp.clone(stop_token_ids=list(dict.fromkeys([*sp.stop_token_ids, *self.extra_eos_token_ids])),
                          stop=list(dict.fromkeys([*(sp.stop or []), *self.extra_stops])))
        ids, text = self._tokenize(prompt)
        if not ids:
            raise ValueError("empty prompt")
        mm_embeds, mm_hash, rope = [], None, None
        if images or videos:
            if self.multimodal is None:
                raise ValueError("this model has no vision tower: images cannot be served")
            ids, mm_embeds, mm_hash, rope = self.multimodal.prepare(ids, images, videos, with_rope=True)
            if len(ids) > self.max_model_len - self.reserve_tokens:
                raise ValueError(f"prompt with images has {len(ids)} tokens; max_model_len is {self.max_model_len}")
        limit = self.max_model_len - self.reserve_tokens
        want = len(ids) + (sp.max_tokens or 0)
        if len(ids) > limit or want > self.max_model_len:
            if len(ids) > limit:
                if not self.auto_truncate_prompt:
                    raise ValueError(f"prompt has {len(ids)} tokens; max_model_len is {self.max_model_len}")
                rope = None     # a truncated prompt keeps consecutive positions
                keep = limit
                if self.truncate_mode == "left":
                    ids = ids[-keep:]
                elif self.truncate_mode == "right":
                    ids = ids[:keep]
                else:
                    ids = ids[: keep // 2] + ids[-(keep - keep // 2):]
            if sp.max_tokens is not None and len(ids) + sp.max_tokens > self.max_model_len:
                sp = sp.clone(max_tokens=max(1, self.max_model_len - len(ids)))
        rid = request_id or f"req-{next(self._ids)}"
        req = EngineRequest(rid, ids, sp, eos_token_id=self.eos_token_id, priority=priority, mm_embeds=mm_embeds,
                            mm_hash=mm_hash)
        if rope is not None:
            req.rope_positions, req.rope_delta = rope
        tr = _Tracked(req, text, IncrementalDetokenizer(self.tokenizer if sp.detokenize else None,
                                                        sp.skip_special_tokens))
        with self._work:
            self._tracked[rid] = tr
            self.scheduler.add_request(req)
            self.metrics.start_request(rid, len(ids))
            self._work.notify_all()
        return rid

    def abort_request(self, request_id: str) -> None:
        with self._work:
            req = self.scheduler.abort_request(request_id)
            tr = self._tracked.get(request_id)
            if req is not None:
                self._return_slot(req)
            if tr is not None:
                tr.finished, tr.finish_reason = True, "abort"
                tr.event.set()

    def _return_slot(self, req: EngineRequest) -> None:
        if req.slot >= 0:
            self._free_slots.append(req.slot)
            req.slot = -1

    # ------------------------------------------------------------------ the step
    def _assign_slots(self, out) -> None:
        for s in out.scheduled:
            if s.request.slot < 0:
                s.request.slot = self._free_slots.pop()
                self.runner._slot_npages[s.request.slot] = 0   # the slot's page mirror belongs to a new request
                self.cache.reset_slot_state(s.request.slot)
                if s.request.sampling_params.needs_penalties:
                    self.runner._ensure_counts()
                    self.runner.reset_slot(s.request.slot, s.request.all_token_ids)

    def _commit(self, out, handle, t_launch) -> int:
        sampled = self.runner.collect(handle)
        finished = self.scheduler.commit_output(out, sampled)
        self._publish(out, sampled, finished)
        self.metrics.record_step(out.total_tokens, len(sampled), time.perf_counter() - t_launch,
                                 self.scheduler.num_running, self.scheduler.num_waiting, self.pool.usage,
                                 self.pool.stats.hit_rate)
        self.last_heartbeat = time.time()
        return out.total_tokens

    def _step_async(self) -> int:
        """schedule(t) -> launch(t) -> read back and commit(t-1) -> book(t): the host work of a step (scheduling,
        batch metadata, detokenisation, stop checks) runs while the device executes the previous launch."""
        with self._lock:
            out = self.scheduler.schedule()
            for r in out.preempted:
                self._return_slot(r)
            handle = None
            if not out.is_empty:
                self._assign_slots(out)
                handle = self.runner.launch(out)
            prev, self._inflight = self._inflight, None
            done = self._commit(*prev) if prev is not None else 0
            if handle is not None:
                self.scheduler.advance_optimistic(out)
                self._inflight = (out, handle, time.perf_counter())
                done += out.total_tokens
            return done

    def step(self) -> int:
        """One schedule -> execute -> update cycle. Returns the number of tokens processed."""
        if self.async_scheduling:
            return self._step_async()
        with self._lock:
            out = self.scheduler.schedule()
            for r in out.preempted:
                self._return_slot(r)
            if out.is_empty:
                return 0
            self._assign_slots(out)
            t0 = time.perf_counter()
            sampled = self.runner.execute(out)
            dt = time.perf_counter() - t0
            finished = self.scheduler.update_from_output(out, sampled)
            self._publish(out, sampled, finished)
            self.metrics.record_step(out.total_tokens, len(sampled), dt, self.scheduler.num_running,
                                     self.scheduler.num_waiting, self.pool.usage, self.pool.stats.hit_rate)
            self.last_heartbeat = time.time()
            return out.total_tokens

    def _publish(self, out, sampled: dict[str, int], finished: list[EngineRequest]) -> None:
        fin = {r.request_id: r for r in finished}
        for s in out.scheduled:
            rid = s.request.request_id
            if rid not in sampled:
                continue
            tr = self._tracked.get(rid)
            if tr is None:
                continue
            tok = sampled[rid]
            req = s.request
            if len(req.output_token_ids) == 1:
                self.metrics.record_first_token(rid)
            delta = tr.detok.push([tok])
            stop_hit = None
            sp = req.sampling_params
            if sp.stop and delta:
                for st in sp.stop:
                    pos = tr.detok.text.find(st, max(0, len(tr.detok.text) - len(delta) - len(st)))
                    if pos >= 0:
                        stop_hit = st
                        cut = pos + (len(st) if sp.include_stop_str_in_output else 0)
                        over = len(tr.detok.text) - cut
                        tr.detok.text = tr.detok.text[:cut]
                        delta = delta[: max(0, len(delta) - over)]
                        break
            with tr.lock:
                tr.pending_delta += delta
                tr.pending_ids.append(tok)
            if stop_hit is not None and rid not in fin:
                req.stop_reason = stop_hit
                self.scheduler.finish_request(req, RequestStatus.FINISHED_STOPPED)
                fin[rid] = req
            tr.event.set()
        for rid, req in fin.items():
            self._return_slot(req)
            tr = self._tracked.get(rid)
            self.metrics.finish_request(rid, len(req.output_token_ids))
            if tr is not None:
                tr.finished = True
                tr.finish_reason = req.status.value
                tr.event.set()

    def _loop(self) -> None:
        while True:
            with self._work:
                while self._running and (self._paused or not (self.scheduler.has_unfinished() or self._inflight)):
                    self.last_heartbeat = time.time()
                    self._work.wait(timeout=0.5)
                if not self._running:
                    return
            try:
                self.step()
                self._errors = 0
            except Exception as e:  # error budget, then fail every in-flight request
                self._errors += 1
                self.metrics.record_error(repr(e))
                if self._errors >= self._max_errors:
                    with self._work:
                        for rid, tr in list(self._tracked.items()):
                            if not tr.finished:
                                self.scheduler.abort_request(rid)
                                tr.finished, tr.finish_reason = True, f"error: {e!r}"
                                tr.event.set()
                    self._errors = 0

    # ------------------------------------------------------------------ user API
    def _snapshot(self, tr: _Tracked, final: bool) -> RequestOutput:
        req = tr.req
        with tr.lock:
            delta, ids = tr.pending_delta, tr.pending_ids
            tr.pending_delta, tr.pending_ids = "", []
        now = time.time()
        n = len(req.output_token_ids)
        elapsed = max(now - tr.start, 1e-9)
        ttft = (req.first_token_time - req.arrival_time) if req.first_token_time else None
        return RequestOutput(
            request_id=req.request_id, prompt=tr.prompt, prompt_token_ids=req.prompt_token_ids,
            outputs=[CompletionOutput(0, tr.detok.text, list(req.output_token_ids),
                                      tr.finish_reason if final else None)],
            finished=final, delta_text=delta, delta_token_ids=ids, tokens_per_second=n / elapsed,
            num_generated_tokens=n, time_to_first_token=ttft, processing_time=elapsed,
            num_cached_tokens=req.num_cached_tokens)

    def generate(self, prompts, sampling_params: SamplingParams | list[SamplingParams] | None = None,
                 request_id: str | list[str] | None = None, use_tqdm: bool = False,
                 images: list | None = None, videos: list | None = None) -> list[RequestOutput]:
        """Blocking batch generation. Works with or without the background thread. ``images`` / ``videos``: the
        images / frame stacks of the prompt (or one list per prompt), one per placeholder token."""
        single = isinstance(prompts, str) or (isinstance(prompts, (list, tuple)) and prompts
                                              and isinstance(prompts[0], int))
        plist = [prompts] if single else list(prompts)
        sps = sampling_params if isinstance(sampling_params, list) else [sampling_params] * len(plist)
        rids = request_id if isinstance(request_id, list) else [request_id] * len(plist)
        if images is None:
            imgs = [None] * len(plist)
        else:
            imgs = [images] if single else list(images)
        vids = [None] * len(plist) if videos is None else ([videos] if single else list(videos))
        ids = [self.add_request(p, sp, rid, images=im, videos=vd)
               for p, sp, rid, im, vd in zip(plist, sps, rids, imgs, vids)]
        self._drive(lambda: all(self._tracked[i].finished for i in ids))
        outs = [self._snapshot(self._tracked.pop(i), True) for i in ids]
        return outs

    def _drive(self, done: tp.Callable[[], bool]) -> None:
        background = self._thread is not None and self._thread.is_alive()
        while not done():
            if background:
                time.sleep(0.001)
            elif self.step() == 0 and not self.scheduler.has_unfinished() and self._inflight is None:
                break

    def stream(self, prompt, sampling_params: SamplingParams | None = None, request_id: str | None = None,
               images: list | None = None, videos: list | None = None) -> tp.Iterator[RequestOutput]:
        """Yields a ``RequestOutput`` whenever new tokens arrive (``delta_text`` holds the increment)."""
        rid = self.add_request(prompt, sampling_params, request_id, images=images, videos=videos)
        tr = self._tracked[rid]
        background = self._thread is not None and self._thread.is_alive()
        try:
            while True:
                if not background:
                    self.step()
                else:
                    tr.event.wait(timeout=1.0)
                tr.event.clear()
                fin = tr.finished
                if tr.pending_ids or fin:
                    yield self._snapshot(tr, fin)
                if fin:
                    break
        finally:
            if not tr.finished:
                self.abort_request(rid)
            self._tracked.pop(rid, None)

    def chat(self, messages: list[dict], sampling_params: SamplingParams | None = None, tools: list | None = None,
             stream: bool = False, chat_template: str | None = None, **template_kwargs):
        if self.tokenizer is None:
            raise ValueError("chat() needs a tokenizer with a chat template")
        images = None
        if self.multimodal is not None:
            images, _ = self.multimodal.extract_media_from_messages(messages)
            if images:
                messages = self.multimodal.normalize_messages(messages)
        prompt = self.tokenizer.apply_chat_template(messages, tools=tools, tokenize=False,
                                                    add_generation_prompt=True, chat_template=chat_template,
                                                    **template_kwargs)
        if stream:
            return self.stream(prompt, sampling_params, images=images or None)
        return self.generate(prompt, sampling_params, images=images or None)[0]

    def get_metrics_summary(self) -> dict:
        m = self.metrics.summary()
        m.update(num_pages=self.cache.num_pages, page_usage=self.pool.usage,
                 prefix_cache_hit_rate=self.pool.stats.hit_rate, runner_timings=dict(self.runner.timings))
        return m

    @property
    def num_pending_requests(self) -> int:
        return self.scheduler.num_waiting

    @property
    def num_running_requests(self) -> int:
        return self.scheduler.num_running

    def __repr__(self):
        return (f"eSurge(name={self.name!r}, max_model_len={self.max_model_len}, max_num_seqs={self.max_num_seqs}, "
                f"pages={self.cache.num_pages}, prefix_caching={self.pool.enable_caching})")
