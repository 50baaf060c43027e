"""``InferenceApiRouter``: an OpenAI-compatible reverse proxy / load balancer over several backends
(easydel/inference/oai_proxies.py). Requests are routed by model name; among the healthy backends that serve the
model the one with the fewest in-flight requests wins (ties: round robin). Streaming bodies are passed through
chunk by chunk. Backends that fail a health probe are skipped until they answer again."""

from __future__ import annotations

import asyncio
import itertools
import time
import typing as tp
from dataclasses import dataclass, field

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse


@dataclass
class Backend:
    url: str
    models: list[str] = field(default_factory=list)
    api_key: str | None = None
    healthy: bool = True
    inflight: int = 0
    failures: int = 0
    last_checked: float = 0.0


class InferenceApiRouter:
    def __init__(self, backends: list[Backend | str | dict], health_interval: float = 10.0, timeout: float = 600.0,
                 max_failures: int = 3):
        self.backends = [b if isinstance(b, Backend) else Backend(**b) if isinstance(b, dict) else Backend(url=b)
                         for b in backends]
        for b in self.backends:
            b.url = b.url.rstrip("/")
        self.health_interval, self.timeout, self.max_failures = health_interval, timeout, max_failures
        self._rr = itertools.count()
        self._session = None
        self.app = self._build()

    async def _client(self):
        import aiohttp

        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout))
        return self._session

    def pick(self, model: str | None) -> Backend:
        cands = [b for b in self.backends if b.healthy and (not model or not b.models or model in b.models)]
        if not cands:
            raise LookupError(f"no healthy backend serves model {model!r}")
        least = min(b.inflight for b in cands)
        cands = [b for b in cands if b.inflight == least]
        return cands[next(self._rr) % len(cands)]

    async def refresh(self, force: bool = False) -> None:
        """Probes ``/health`` and, for backends without a model list, ``/v1/models``."""
        sess = await self._client()
        now = time.time()
        for b in self.backends:
            if not force and now - b.last_checked < self.health_interval:
                continue
            b.last_checked = now
            try:
                async with sess.get(b.url + "/health") as r:
                    ok = r.status == 200
                if ok and not b.models:
                    async with sess.get(b.url + "/v1/models", headers=self._headers(b, {})) as r:
                        if r.status == 200:
                            b.models = [m["id"] for m in (await r.json()).get("data", [])]
                b.healthy, b.failures = ok, 0 if ok else b.failures + 1
            except Exception:  # noqa: BLE001
                b.failures += 1
                b.healthy = b.failures < self.max_failures

    @staticmethod
    def _headers(b: Backend, incoming: tp.Mapping[str, str]) -> dict:
        h = {k: v for k, v in incoming.items() if k.lower() in ("content-type", "accept", "authorization", "x-api-key")}
        if b.api_key:
            h["Authorization"] = f"Bearer {b.api_key}"
        return h

    def _build(self) -> FastAPI:
        app = FastAPI(title="eSurge router")
        router = self

        @app.get("/health")
        async def health():
            await router.refresh()
            return {"status": "ok" if any(b.healthy for b in router.backends) else "degraded",
                    "backends": [{"url": b.url, "healthy": b.healthy, "inflight": b.inflight, "models": b.models}
                                 for b in router.backends]}

        @app.get("/v1/models")
        async def models():
            await router.refresh()
            seen, data = set(), []
            for b in router.backends:
                for m in b.models:
                    if b.healthy and m not in seen:
                        seen.add(m)
                        data.append({"id": m, "object": "model", "owned_by": "easydel"})
            return {"object": "list", "data": data}

        async def forward(path: str, request: Request):
            body = await request.json()
            await router.refresh()
            try:
                b = router.pick(body.get("model"))
            except LookupError as e:
                raise HTTPException(status_code=503, detail=str(e)) from e
            sess = await router._client()
            b.inflight += 1
            try:
                resp = await sess.post(b.url + path, json=body, headers=router._headers(b, request.headers))
            except Exception as e:  # noqa: BLE001
                b.inflight -= 1
                b.failures += 1
                b.healthy = b.failures < router.max_failures
                raise HTTPException(status_code=502, detail=f"backend {b.url} failed: {e}") from e
            if body.get("stream"):
                async def relay():
                    try:
                        async for chunk in resp.content.iter_any():
                            yield chunk
                    finally:
                        resp.release()
                        b.inflight -= 1

                return StreamingResponse(relay(), status_code=resp.status, media_type="text/event-stream")
            try:
                data = await resp.json()
            finally:
                resp.release()
                b.inflight -= 1
            return JSONResponse(data, status_code=resp.status)

        @app.post("/v1/chat/completions")
        async def chat(request: Request):
            return await forward("/v1/chat/completions", request)

        @app.post("/v1/completions")
        async def completions(request: Request):
            return await forward("/v1/completions", request)

        @app.post("/v1/responses")
        async def responses(request: Request):
            return await forward("/v1/responses", request)

        @app.on_event("shutdown")
        async def close():
            if router._session is not None and not router._session.closed:
                await router._session.close()

        return app

    def run(self, host: str = "0.0.0.0", port: int = 8080) -> None:
        import uvicorn

        uvicorn.run(self.app, host=host, port=port)
