"""Continuous-batching scheduler with a per-step token budget.

Same policy as easydel/inference/esurge/scheduler/scheduler.py:374-860: running requests are
scheduled first (one token each while decoding, or the next chunk of an unfinished prefill), then
waiting requests are admitted FCFS (or by priority) while the token budget, the sequence limit
and the page pool allow; long prefills are chunked to ``long_prefill_token_threshold`` /
the remaining budget; when pages run out the most recently admitted running request is
preempted (its pages are released and it re-enters the waiting queue, keeping its generated
tokens). Prefix-cache hits are resolved on admission: matching full pages are shared, and the
request starts with ``num_computed_tokens`` equal to the cached length.
"""

from __future__ import annotations

import collections
import enum
import itertools
import time
import typing as tp
from dataclasses import dataclass, field

from ..sampling_params import SamplingParams
from .kv_manager import KVCacheCoordinator
from .page_pool import PagePool, hash_request_pages


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED_STOPPED = "stop"
    FINISHED_LENGTH = "length"
    FINISHED_ABORTED = "abort"

    @property
    def finished(self) -> bool:
        return self in (RequestStatus.FINISHED_STOPPED, RequestStatus.FINISHED_LENGTH,
                        RequestStatus.FINISHED_ABORTED)


_arrival = itertools.count()


EngineRequestStatus = RequestStatus      # the name the public namespace uses


@dataclass
class EngineRequest:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    eos_token_id: int | None = None
    arrival_time: float = field(default_factory=time.time)
    priority: int = 0
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    num_computed_tokens: int = 0          # tokens whose KV is in the cache
    num_cached_tokens: int = 0            # prefix-cache hit length at (last) admission
    pages: list[int] = field(default_factory=list)              # page list of cache group 0
    group_pages: list[list[int]] = field(default_factory=list)  # page lists of the other cache groups, same indexing
    page_hashes: list[bytes] = field(default_factory=list)
    num_registered_pages: int = 0
    pages_epoch: int = 0                  # bumped whenever entries of a page list change in place (window release)
    slot: int = -1                        # row in the runner's persistent per-sequence buffers
    order: int = field(default_factory=lambda: next(_arrival))
    first_token_time: float | None = None
    finish_time: float | None = None
    num_preemptions: int = 0
    stop_reason: tp.Any = None
    # images: (offset of the first placeholder token in the prompt, projected features [rows, hidden] on the device)
    mm_embeds: list = field(default_factory=list)
    mm_hash: tp.Any = None                # joins the page hashes: same tokens + other images = other pages
    # three-stream rotary models: [3, prompt length] int32 rotary positions of the prompt (vision tokens carry grid
    # coordinates) and the offset a generated token's rotary position has from its index; None = index everywhere
    rope_positions: tp.Any = None
    rope_delta: int = 0
    # asynchronous scheduling: the request reached its length limit with a token that is still on the device;
    # it is not scheduled again and finishes when that token is committed
    finishing: bool = False

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def max_total_tokens(self) -> int:
        return self.num_prompt_tokens + (self.sampling_params.max_tokens or 0)


#: stands in ``output_token_ids`` for a token that was sampled on the device and not read back yet
PLACEHOLDER_TOKEN = -1


@dataclass
class ScheduledRequest:
    request: EngineRequest
    num_new_tokens: int            # tokens fed to the model this step
    start: int                     # index (in all_token_ids) of the first fed token
    samples: bool                  # True when this step produces the next token for the request
    out_index: int = -1            # asynchronous scheduling: where in output_token_ids this step's token goes


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest]
    preempted: list[EngineRequest]
    total_tokens: int
    num_decode: int

    @property
    def is_empty(self) -> bool:
        return not self.scheduled


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 2048
    max_model_len: int = 8192
    long_prefill_token_threshold: int | None = None
    policy: str = "fcfs"            # "fcfs" | "priority"
    enable_chunked_prefill: bool = True


class Scheduler:
    def __init__(self, config: SchedulerConfig, pool: "PagePool | KVCacheCoordinator", page_size: int = 128):
        # one pool = one full-attention group; a coordinator carries one pool per cache group
        self.kv = pool if isinstance(pool, KVCacheCoordinator) else KVCacheCoordinator.single(pool, page_size)
        self.config, self.pool, self.page_size = config, self.kv.pool, page_size
        self.waiting: collections.deque[EngineRequest] = collections.deque()
        self.running: list[EngineRequest] = []
        self.num_preemptions = 0          # requests pushed back to the waiting queue since the scheduler was built
        self.requests: dict[str, EngineRequest] = {}
        self.finished_ids: list[str] = []

    # ------------------------------------------------------------------ queue management
    def add_request(self, req: EngineRequest) -> None:
        if req.num_prompt_tokens >= self.config.max_model_len:
            raise ValueError(f"prompt of {req.num_prompt_tokens} tokens does not fit max_model_len "
                             f"{self.config.max_model_len}")
        self.requests[req.request_id] = req
        req.status = RequestStatus.WAITING
        if self.config.policy == "priority":
            items = sorted([*self.waiting, req], key=lambda r: (r.priority, r.order))
            self.waiting = collections.deque(items)
        else:
            self.waiting.append(req)

    def abort_request(self, request_id: str) -> EngineRequest | None:
        req = self.requests.get(request_id)
        if req is None or req.status.finished:
            return None
        self._finish(req, RequestStatus.FINISHED_ABORTED)
        return req

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_running(self) -> int:
        return len(self.running)

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)

    # ------------------------------------------------------------------ pages
    def _try_allocate(self, req: EngineRequest, upto_tokens: int) -> bool:
        """Pages for ``upto_tokens`` tokens in every cache group, or nothing. Window-bounded groups first give back
        the pages no later query of this request can reach (every launched step is ahead of the next one on the
        stream, so a page freed here is not read again before its new owner writes it)."""
        if self.kv.remove_skipped(req):
            req.pages_epoch += 1
        return self.kv.try_allocate(req, upto_tokens)

    def _release(self, req: EngineRequest) -> None:
        self.kv.release(req)
        req.num_registered_pages = 0

    def _preempt(self, req: EngineRequest) -> None:
        self._release(req)
        req.status = RequestStatus.PREEMPTED
        req.num_computed_tokens = 0
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)

    def _admit_with_prefix(self, req: EngineRequest) -> None:
        """Shares the cached full pages that match the request's token prefix."""
        tokens = req.all_token_ids
        req.page_hashes = hash_request_pages(tokens, self.page_size, req.mm_hash)
        # never serve the whole request from cache: the last token must be recomputed to produce logits
        usable = req.page_hashes[: max(0, (len(tokens) - 1) // self.page_size)]
        n_hit = self.kv.admit_with_prefix(req, usable)
        req.num_registered_pages = n_hit
        req.num_cached_tokens = n_hit * self.page_size
        req.num_computed_tokens = req.num_cached_tokens

    def _register_full_pages(self, req: EngineRequest) -> None:
        """Publishes pages that became full (and whose tokens are final) for prefix reuse."""
        if not self.pool.enable_caching:
            return
        known = req.num_tokens
        if req.output_token_ids and req.output_token_ids[-1] == PLACEHOLDER_TOKEN:
            known -= 1          # that token is still on the device: its page cannot be hashed yet
        full = min(req.num_computed_tokens, known) // self.page_size
        if full <= req.num_registered_pages:
            return
        tokens = req.all_token_ids
        if len(req.page_hashes) < full:
            req.page_hashes = hash_request_pages(tokens[: full * self.page_size], self.page_size, req.mm_hash)
        for i in range(req.num_registered_pages, full):
            self.kv.register(req, i, req.page_hashes[i])
        req.num_registered_pages = full

    # ------------------------------------------------------------------ the step
    def schedule(self) -> SchedulerOutput:
        cfg = self.config
        budget = cfg.max_num_batched_tokens
        scheduled: list[ScheduledRequest] = []
        preempted: list[EngineRequest] = []
        chunk_cap = cfg.long_prefill_token_threshold or budget

        # 1) running requests, oldest first
        i = 0
        running = sorted(self.running, key=lambda r: r.order)
        while i < len(running) and budget > 0:
            req = running[i]
            if req.status != RequestStatus.RUNNING or req.finishing:
                i += 1
                continue
            remaining = req.num_tokens - req.num_computed_tokens
            n = min(remaining, budget, chunk_cap if remaining > 1 else 1)
            if n <= 0:
                i += 1
                continue
            while not self._try_allocate(req, req.num_computed_tokens + n):
                # free pages by preempting the newest running request (possibly this one)
                victim = max((r for r in self.running if r.status == RequestStatus.RUNNING and
                              (not r.finishing or r is req)), key=lambda r: r.order)
                self._preempt(victim)
                preempted.append(victim)
                scheduled = [s for s in scheduled if s.request is not victim]
                if victim is req:
                    break
            if req.status != RequestStatus.RUNNING:
                i += 1
                continue
            scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens,
                                              req.num_computed_tokens + n == req.num_tokens))
            budget -= n
            i += 1

        # 2) admit waiting requests while nothing was preempted this step
        while self.waiting and budget > 0 and not preempted and len(self.running) < cfg.max_num_seqs:
            req = self.waiting[0]
            if not req.pages and req.num_computed_tokens == 0:
                self._admit_with_prefix(req)
            remaining = req.num_tokens - req.num_computed_tokens
            n = min(remaining, budget, chunk_cap)
            if n < remaining and not cfg.enable_chunked_prefill:
                # without chunking a prompt must fit the budget in one go
                if remaining > cfg.max_num_batched_tokens:
                    n = min(remaining, cfg.max_num_batched_tokens)
                else:
                    self._release(req)
                    req.num_computed_tokens = 0
                    break
            if not self._try_allocate(req, req.num_computed_tokens + n):
                self._release(req)
                req.num_computed_tokens = 0
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens,
                                              req.num_computed_tokens + n == req.num_tokens))
            budget -= n

        # decode-first ordering: single-token steps of running requests lead the batch
        scheduled.sort(key=lambda s: (s.num_new_tokens > 1, s.request.order))
        num_decode = sum(1 for s in scheduled if s.num_new_tokens == 1)
        return SchedulerOutput(scheduled, preempted, sum(s.num_new_tokens for s in scheduled), num_decode)

    # ------------------------------------------------------------------ asynchronous scheduling
    # The engine launches step t before it has read the tokens of step t-1 (the reference's ``AsyncScheduler``,
    # easydel/inference/esurge/scheduler/async_scheduler.py:68). Between launch and read-back a sampled token is a
    # placeholder in ``output_token_ids``; the runner feeds the real value from its device-side token table.
    def advance_optimistic(self, out: SchedulerOutput) -> None:
        """Books a launched step: computed-token counts move on and every sampling row gets a placeholder token.
        Length limits are known without the token, so a request that reaches one stops being scheduled now."""
        for s in out.scheduled:
            req = s.request
            if req.status != RequestStatus.RUNNING:
                continue
            req.num_computed_tokens += s.num_new_tokens
            if not s.samples:
                continue
            s.out_index = len(req.output_token_ids)
            req.output_token_ids.append(PLACEHOLDER_TOKEN)
            sp = req.sampling_params
            if (sp.max_tokens is not None and len(req.output_token_ids) >= sp.max_tokens) or \
                    req.num_tokens >= self.config.max_model_len:
                req.finishing = True

    def commit_output(self, out: SchedulerOutput, sampled: dict[str, int]) -> list[EngineRequest]:
        """Fills in the tokens of a step booked by :meth:`advance_optimistic` and applies the stop conditions.
        A request that stops on a token (EOS, stop id) may already be part of the next, launched step: that row's
        result is dropped when its turn to be committed comes, because the request is no longer running."""
        finished = []
        now = time.time()
        for s in out.scheduled:
            req = s.request
            if req.status.finished:
                continue               # stopped or aborted meanwhile: the row's result is dropped
            running = req.status == RequestStatus.RUNNING
            if not s.samples or s.out_index < 0:
                if running:
                    self._register_full_pages(req)
                continue
            if req.request_id not in sampled or s.out_index >= len(req.output_token_ids):
                continue
            # a request preempted after the launch keeps its token: it was sampled from a complete context
            tok = int(sampled[req.request_id])
            req.output_token_ids[s.out_index] = tok
            if req.first_token_time is None:
                req.first_token_time = now
            status = self._check_stop_at(req, tok, s.out_index + 1)
            if status is not None:
                del req.output_token_ids[s.out_index + 1:]
                if running:
                    self._register_full_pages(req)
                self._finish(req, status)
                finished.append(req)
                continue
            if running:
                self._register_full_pages(req)
        return finished

    def _check_stop_at(self, req: EngineRequest, tok: int, n_out: int) -> RequestStatus | None:
        sp = req.sampling_params
        if n_out >= sp.min_tokens:
            if not sp.ignore_eos and req.eos_token_id is not None and tok == req.eos_token_id:
                req.stop_reason = "eos"
                return RequestStatus.FINISHED_STOPPED
            if tok in sp.stop_token_ids:
                req.stop_reason = tok
                return RequestStatus.FINISHED_STOPPED
        if sp.max_tokens is not None and n_out >= sp.max_tokens:
            return RequestStatus.FINISHED_LENGTH
        if req.num_prompt_tokens + n_out >= self.config.max_model_len:
            return RequestStatus.FINISHED_LENGTH
        return None

    # ------------------------------------------------------------------ after the model ran
    def update_from_output(self, out: SchedulerOutput, sampled: dict[str, int]) -> list[EngineRequest]:
        """Advances computed-token counts, appends sampled tokens, applies stop conditions.
        Returns the requests that finished in this step."""
        finished = []
        now = time.time()
        for s in out.scheduled:
            req = s.request
            if req.status != RequestStatus.RUNNING:
                continue
            req.num_computed_tokens += s.num_new_tokens
            if s.samples and req.request_id in sampled:
                tok = int(sampled[req.request_id])
                req.output_token_ids.append(tok)
                if req.first_token_time is None:
                    req.first_token_time = now
                status = self._check_stop(req, tok)
                if status is not None:
                    self._register_full_pages(req)
                    self._finish(req, status)
                    finished.append(req)
                    continue
            self._register_full_pages(req)
        return finished

    def _check_stop(self, req: EngineRequest, tok: int) -> RequestStatus | None:
        sp = req.sampling_params
        n_out = len(req.output_token_ids)
        if n_out >= sp.min_tokens:
            if not sp.ignore_eos and req.eos_token_id is not None and tok == req.eos_token_id:
                req.stop_reason = "eos"
                return RequestStatus.FINISHED_STOPPED
            if tok in sp.stop_token_ids:
                req.stop_reason = tok
                return RequestStatus.FINISHED_STOPPED
        if sp.max_tokens is not None and n_out >= sp.max_tokens:
            return RequestStatus.FINISHED_LENGTH
        if req.num_tokens >= self.config.max_model_len:
            return RequestStatus.FINISHED_LENGTH
        return None

    def finish_request(self, req: EngineRequest, status: RequestStatus = RequestStatus.FINISHED_STOPPED) -> None:
        """Lets the engine stop a request for reasons the scheduler cannot see (stop strings)."""
        if not req.status.finished:
            self._finish(req, status)

    def _finish(self, req: EngineRequest, status: RequestStatus) -> None:
        if req in self.running:
            self.running.remove(req)
        try:
            self.waiting.remove(req)
        except ValueError:
            pass
        self._release(req)
        req.status = status
        req.finish_time = time.time()
        self.finished_ids.append(req.request_id)
        self.requests.pop(req.request_id, None)
