"""Engine metrics: TTFT, per-request latency, token throughput, scheduler / cache gauges.

Counterpart of ``MetricsCollector`` (easydel/inference/esurge/metrics.py:247-749). TTFT is measured from
``start_request`` to ``record_first_token`` like the reference (:331-366). ``prometheus_text`` renders the
gauges in the Prometheus exposition format for the ``/metrics`` endpoint.
"""

from __future__ import annotations

import statistics
import threading
import time
from dataclasses import dataclass, field


@dataclass
class _Req:
    start: float
    prompt_tokens: int
    first_token: float | None = None
    end: float | None = None
    generated: int = 0


def _pct(xs: list[float], q: float) -> float | None:
    if not xs:
        return None
    xs = sorted(xs)
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


class MetricsCollector:
    def __init__(self, history: int = 100000):
        self.lock = threading.Lock()
        self.active: dict[str, _Req] = {}
        self.done: list[_Req] = []
        self.history = history
        self.total_steps = 0
        self.total_tokens_processed = 0
        self.total_tokens_generated = 0
        self.total_step_time = 0.0
        self.errors: list[str] = []
        self.gauges = {"running": 0, "waiting": 0, "page_usage": 0.0, "prefix_hit_rate": 0.0}
        self.started = time.time()

    def start_request(self, rid: str, prompt_tokens: int) -> None:
        with self.lock:
            self.active[rid] = _Req(time.time(), prompt_tokens)

    def record_first_token(self, rid: str) -> None:
        with self.lock:
            r = self.active.get(rid)
            if r is not None and r.first_token is None:
                r.first_token = time.time()

    def finish_request(self, rid: str, generated: int) -> None:
        with self.lock:
            r = self.active.pop(rid, None)
            if r is None:
                return
            r.end, r.generated = time.time(), generated
            self.done.append(r)
            if len(self.done) > self.history:
                del self.done[: len(self.done) - self.history]

    def record_step(self, tokens: int, sampled: int, dt: float, running: int, waiting: int, page_usage: float,
                    hit_rate: float) -> None:
        with self.lock:
            self.total_steps += 1
            self.total_tokens_processed += tokens
            self.total_tokens_generated += sampled
            self.total_step_time += dt
            self.gauges.update(running=running, waiting=waiting, page_usage=page_usage, prefix_hit_rate=hit_rate)

    def record_error(self, msg: str) -> None:
        with self.lock:
            self.errors.append(msg)
            del self.errors[:-50]

    def summary(self) -> dict:
        with self.lock:
            ttft = [r.first_token - r.start for r in self.done if r.first_token]
            lat = [r.end - r.start for r in self.done if r.end]
            tpot = [(r.end - r.first_token) / (r.generated - 1) for r in self.done
                    if r.first_token and r.end and r.generated > 1]
            wall = time.time() - self.started
            return {
                "requests_completed": len(self.done), "requests_active": len(self.active),
                "total_steps": self.total_steps, "tokens_processed": self.total_tokens_processed,
                "tokens_generated": self.total_tokens_generated,
                "output_tokens_per_second": self.total_tokens_generated / max(self.total_step_time, 1e-9),
                "output_tokens_per_second_wall": self.total_tokens_generated / max(wall, 1e-9),
                "avg_step_ms": 1e3 * self.total_step_time / max(self.total_steps, 1),
                "ttft_p50": _pct(ttft, 0.5), "ttft_p99": _pct(ttft, 0.99), "ttft_mean": statistics.fmean(ttft) if ttft else None,
                "tpot_p50": _pct(tpot, 0.5), "tpot_p99": _pct(tpot, 0.99),
                "latency_p50": _pct(lat, 0.5), "latency_p99": _pct(lat, 0.99),
                "errors": list(self.errors), **self.gauges,
            }

    def prometheus_text(self, prefix: str = "esurge") -> str:
        s = self.summary()
        lines = []
        for k, v in s.items():
            if isinstance(v, (int, float)) and v is not None:
                lines.append(f"# TYPE {prefix}_{k} gauge")
                lines.append(f"{prefix}_{k} {float(v)}")
        return "\n".join(lines) + "\n"
