"""Data-parallel serving: several engine replicas behind one front, KV pages local to the replica that admitted a request.

The reference shards the page tensor over its ``dp`` axis inside one SPMD engine and pins every request to the shard
that admitted it (easydel/inference/esurge/core/dp_sharding.py:26-60, the shard-aware admission in
easydel/inference/esurge/scheduler/scheduler.py:417-491, the ``ATTN_DP`` axis of easydel/axis.py:24-98). With one
process per GPU the same arrangement is one engine per data-parallel group (a single GPU or a tensor-parallel group),
each with its own page pools, and this router in front of them:

* a request is admitted by the replica that already caches the longest prefix of its prompt, ties broken towards the
  replica with the most free pages and the fewest queued tokens (so shared system prompts stay where their pages are);
* its pages, slots and recurrent state never leave that replica; aborts and results are routed by request id;
* attention therefore runs data-parallel (every replica attends over its own requests only) while the replicas'
  weights may be sharded by tensor / expert parallelism inside each group: the layout the reference calls attention
  data parallelism.

Replicas in the same process are stepped round-robin by :meth:`step`; replicas in other processes run their own
engine loops and are reached through the same interface by the API router (``inference/oai_proxies.py``).
"""

from __future__ import annotations

import itertools
import typing as tp

from ..sampling_params import SamplingParams
from .page_pool import hash_request_pages


def pages_per_dp_shard(num_pages: int, dp_size: int) -> int | None:
    """Pages each of ``dp_size`` replicas gets out of a common budget (every replica keeps its own null page)."""
    dp_size = max(1, int(dp_size))
    if num_pages < 2 * dp_size:
        return None
    return num_pages // dp_size


class DataParallelEngine:
    def __init__(self, engines: tp.Sequence, policy: str = "prefix_affinity"):
        if not engines:
            raise ValueError("need at least one engine replica")
        if policy not in ("prefix_affinity", "least_loaded", "round_robin"):
            raise ValueError(f"unknown routing policy {policy!r}")
        self.engines = list(engines)
        self.policy = policy
        self.owner: dict[str, int] = {}
        self._rr = itertools.count()
        self._ids = itertools.count()
        self.routed = [0] * len(self.engines)

    # ------------------------------------------------------------------ routing
    def _load(self, i: int) -> tuple[float, int]:
        eng = self.engines[i]
        sch = eng.scheduler
        queued = sum(r.num_tokens - r.num_computed_tokens for r in sch.waiting)
        return (-min(m.pool.num_free / max(1, m.pool.num_pages - 1) for m in eng.kv.managers),
                queued + len(sch.running))

    def _prefix_pages(self, i: int, hashes) -> int:
        eng = self.engines[i]
        if not eng.kv.enable_caching or not hashes:
            return 0
        n = len(hashes)
        for m in eng.kv.managers:
            if m.bounded:
                continue
            k = 0
            cached = m.pool.cached
            while k < n and hashes[k] in cached:
                k += 1
            n = k
        while n > 0 and not all(m.holds(hashes, n) for m in eng.kv.managers if m.bounded):
            n -= 1
        return n

    def choose(self, prompt_token_ids: tp.Sequence[int]) -> int:
        n = len(self.engines)
        if n == 1:
            return 0
        if self.policy == "round_robin":
            return next(self._rr) % n
        best = min(range(n), key=self._load)
        if self.policy == "least_loaded":
            return best
        page = self.engines[0].page_size
        hashes = hash_request_pages(list(prompt_token_ids), page)[: max(0, (len(prompt_token_ids) - 1) // page)]
        hits = [self._prefix_pages(i, hashes) for i in range(n)]
        top = max(hits)
        if top == 0:
            return best
        return min((i for i in range(n) if hits[i] == top), key=self._load)

    # ------------------------------------------------------------------ engine surface
    def add_request(self, prompt, sampling_params: SamplingParams | None = None, request_id: str | None = None,
                    **kw) -> str:
        eng0 = self.engines[0]
        ids = prompt if not isinstance(prompt, str) else eng0.tokenizer(prompt)["input_ids"]
        i = self.choose(ids)
        rid = request_id or f"dp-{next(self._ids)}"
        self.engines[i].add_request(ids, sampling_params, request_id=rid, **kw)
        self.owner[rid] = i
        self.routed[i] += 1
        return rid

    def shard_of(self, request_id: str) -> int:
        return self.owner[request_id]

    def abort_request(self, request_id: str) -> None:
        i = self.owner.get(request_id)
        if i is not None:
            self.engines[i].abort_request(request_id)

    def has_unfinished(self) -> bool:
        return any(e.scheduler.has_unfinished() or getattr(e, "_inflight", None) is not None for e in self.engines)

    def step(self) -> None:
        """One engine step on every replica that has work (launch order = replica order; with asynchronous
        scheduling the replicas' device work overlaps)."""
        for e in self.engines:
            if e.scheduler.has_unfinished() or getattr(e, "_inflight", None) is not None:
                e.step()

    def generate(self, prompts, sampling_params: SamplingParams | None = None):
        single = bool(prompts) and isinstance(prompts[0], int)
        plist = [prompts] if single or isinstance(prompts, str) else list(prompts)
        rids = [self.add_request(p, sampling_params) for p in plist]
        while self.has_unfinished():
            self.step()
        outs = []
        for r in rids:
            eng = self.engines[self.owner[r]]
            outs.append(eng._snapshot(eng._tracked.pop(r), True))
        return outs[0] if single or isinstance(prompts, str) else outs

    def get_metrics_summary(self) -> dict:
        per = [e.get_metrics_summary() for e in self.engines]
        out = {"replicas": len(per), "requests_routed": list(self.routed)}
        for k in ("requests_completed", "tokens_generated"):
            out[k] = sum(p.get(k, 0) for p in per)
        out["page_usage"] = [p.get("page_usage") for p in per]
        out["prefix_cache_hit_rate"] = [p.get("prefix_cache_hit_rate") for p in per]
        return out

    def close(self) -> None:
        for e in self.engines:
            e.close()
