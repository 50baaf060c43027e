"""Metrics export and console monitoring for the engine (easydel/inference/esurge/monitoring.py, dashboard.py).

``PrometheusMetrics`` mirrors the engine's ``MetricsCollector`` into ``prometheus_client`` gauges / counters /
histograms and can serve them on an HTTP port; ``RichConsoleMonitor`` prints a one-line status at an interval;
``eSurgeMonitoringServer`` bundles both and can write a Prometheus scrape config plus a Grafana dashboard JSON
(provisioning files only: nothing is launched here).
"""

from __future__ import annotations

import json
import os
import threading
import time
import typing as tp


class PrometheusMetrics:
    def __init__(self, engine, namespace: str = "esurge", registry=None):
        import prometheus_client as pc

        self.engine = engine
        self.registry = registry or pc.CollectorRegistry()
        g = lambda n, d: pc.Gauge(f"{namespace}_{n}", d, ["model"], registry=self.registry)  # noqa: E731
        self.running = g("running_requests", "requests being decoded")
        self.waiting = g("waiting_requests", "requests waiting for admission")
        self.page_usage = g("kv_page_usage", "fraction of KV pages in use")
        self.hit_rate = g("prefix_cache_hit_rate", "prefix cache hit rate")
        self.tps = g("output_tokens_per_second", "recent output token throughput")
        self.ttft = g("ttft_p50_seconds", "median time to first token")
        self.tokens = pc.Counter(f"{namespace}_generated_tokens", "tokens generated", ["model"],
                                 registry=self.registry)
        self.requests = pc.Counter(f"{namespace}_finished_requests", "requests finished", ["model"],
                                   registry=self.registry)
        self.step_time = pc.Histogram(f"{namespace}_step_seconds", "engine step latency", ["model"],
                                      buckets=(0.001, 0.002, 0.005, 0.01, 0.02, 0.05, 0.1, 0.25, 0.5, 1.0),
                                      registry=self.registry)
        self._last = {"tokens": 0, "requests": 0, "steps": 0}
        self._server = None

    def update(self) -> dict:
        e = self.engine
        name = e.name
        s = e.get_metrics_summary()
        self.running.labels(name).set(e.num_running_requests)
        self.waiting.labels(name).set(e.num_pending_requests)
        self.page_usage.labels(name).set(s.get("page_usage", 0.0))
        self.hit_rate.labels(name).set(s.get("prefix_cache_hit_rate", 0.0))
        self.tps.labels(name).set(s.get("tokens_per_second", s.get("output_tokens_per_second", 0.0)) or 0.0)
        if s.get("ttft_p50") is not None:
            self.ttft.labels(name).set(s["ttft_p50"])
        tok = int(s.get("total_generated_tokens", s.get("generated_tokens", 0)) or 0)
        req = int(s.get("finished_requests", s.get("requests_finished", 0)) or 0)
        if tok > self._last["tokens"]:
            self.tokens.labels(name).inc(tok - self._last["tokens"])
            self._last["tokens"] = tok
        if req > self._last["requests"]:
            self.requests.labels(name).inc(req - self._last["requests"])
            self._last["requests"] = req
        if s.get("avg_step_time"):
            self.step_time.labels(name).observe(s["avg_step_time"])
        return s

    def render(self) -> bytes:
        import prometheus_client as pc

        self.update()
        return pc.generate_latest(self.registry)

    def start_http_server(self, port: int = 9090, addr: str = "0.0.0.0"):
        import prometheus_client as pc

        self._server = pc.start_http_server(port, addr=addr, registry=self.registry)
        return self._server


class RichConsoleMonitor:
    def __init__(self, engine, interval: float = 2.0, out: tp.Callable[[str], None] = print):
        self.engine, self.interval, self.out = engine, interval, out
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def line(self) -> str:
        e = self.engine
        s = e.get_metrics_summary()
        return (f"[{e.name}] running={e.num_running_requests} waiting={e.num_pending_requests} "
                f"pages={s.get('page_usage', 0.0):.0%} prefix_hit={s.get('prefix_cache_hit_rate', 0.0):.0%} "
                f"tok/s={s.get('tokens_per_second', 0.0) or 0.0:.0f}")

    def start(self):
        def run():
            while not self._stop.wait(self.interval):
                self.out(self.line())

        self._thread = threading.Thread(target=run, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()


class eSurgeMonitoringServer:
    def __init__(self, engine, prometheus_port: int = 9090, console: bool = False, console_interval: float = 2.0):
        self.metrics = PrometheusMetrics(engine)
        self.port = prometheus_port
        self.console = RichConsoleMonitor(engine, console_interval) if console else None
        self._updater: threading.Thread | None = None
        self._stop = threading.Event()

    def start(self, update_interval: float = 1.0):
        self.metrics.start_http_server(self.port)
        if self.console:
            self.console.start()

        def run():
            while not self._stop.wait(update_interval):
                self.metrics.update()

        self._updater = threading.Thread(target=run, daemon=True)
        self._updater.start()
        return self

    def stop(self):
        self._stop.set()
        if self.console:
            self.console.stop()

    def write_provisioning(self, directory: str, scrape_target: str | None = None) -> dict[str, str]:
        """Writes ``prometheus.yml`` and ``grafana_dashboard.json`` for this exporter."""
        os.makedirs(directory, exist_ok=True)
        target = scrape_target or f"localhost:{self.port}"
        prom = os.path.join(directory, "prometheus.yml")
        with open(prom, "w") as f:
            f.write("global:\n  scrape_interval: 5s\nscrape_configs:\n  - job_name: esurge\n    static_configs:\n"
                    f"      - targets: ['{target}']\n")
        panels = [{"type": "timeseries", "title": t, "targets": [{"expr": q}], "gridPos": {"h": 8, "w": 12,
                   "x": 12 * (i % 2), "y": 8 * (i // 2)}}
                  for i, (t, q) in enumerate([
                      ("Output tokens / s", "esurge_output_tokens_per_second"),
                      ("Running / waiting", "esurge_running_requests or esurge_waiting_requests"),
                      ("KV page usage", "esurge_kv_page_usage"),
                      ("Prefix cache hit rate", "esurge_prefix_cache_hit_rate"),
                      ("TTFT p50 (s)", "esurge_ttft_p50_seconds"),
                      ("Step latency", "rate(esurge_step_seconds_sum[1m]) / rate(esurge_step_seconds_count[1m])")])]
        dash = os.path.join(directory, "grafana_dashboard.json")
        with open(dash, "w") as f:
            json.dump({"title": "eSurge", "schemaVersion": 39, "refresh": "5s", "panels": panels,
                       "time": {"from": "now-15m", "to": "now"}}, f, indent=1)
        return {"prometheus": prom, "grafana": dash}
