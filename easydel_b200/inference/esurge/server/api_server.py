"""OpenAI-compatible HTTP server over one or more eSurge engines.

Endpoints (easydel/inference/inference_engine_interface.py:464-610 and esurge/server/api_server.py):
``/v1/chat/completions``, ``/v1/completions``, ``/v1/responses``, ``/v1/models``, ``/v1/models/{id}``, ``/health``,
``/metrics``, ``/v1/tools``, ``/v1/tools/execute``, admin ``/v1/admin/keys*`` and ``/v1/admin/audit-logs``.
Streaming uses server-sent events; a client disconnect aborts the request in the engine. Tool calls and
reasoning text are split out of the model text by the parsers in ``inference.tools`` / ``inference.reasoning``.

The engine's scheduler thread produces tokens; request handlers run on the asyncio loop and pull the engine's
blocking iterators through a thread so that slow clients never stall the scheduler.
"""

from __future__ import annotations

import asyncio
import json
import time
import typing as tp

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ...openai_api_modules import (ChatCompletionRequest, ChatCompletionResponse, ChatCompletionResponseChoice,
                                   ChatCompletionStreamResponse, ChatCompletionStreamResponseChoice, ChatMessage,
                                   CompletionRequest, CompletionResponse, CompletionResponseChoice, DeltaMessage,
                                   ModelCard, ModelList, ResponsesRequest, ResponsesResponse, ToolCall,
                                   ToolExecuteRequest, UsageInfo, sse)
from ...reasoning import DelegatingParser, ReasoningParserManager, detect_reasoning_parser
from ...stream_protocol import ResponsesStreamBuilder, sse_frame
from ...tools import ToolParserManager, detect_tool_parser


def _usage(out) -> UsageInfo:
    p = len(out.prompt_token_ids)
    return UsageInfo(prompt_tokens=p, completion_tokens=out.num_generated_tokens,
                     total_tokens=p + out.num_generated_tokens, tokens_per_second=out.tokens_per_second,
                     processing_time=out.processing_time, time_to_first_token=out.time_to_first_token,
                     cached_tokens=out.num_cached_tokens)


def _finish_reason(out, has_tools: bool) -> str:
    if has_tools:
        return "tool_calls"
    r = out.outputs[0].finish_reason if out.outputs else None
    return {"length": "length", "abort": "stop", None: "stop"}.get(r, "stop" if r != "length" else "length")


class eSurgeApiServer:
    def __init__(self, engines: tp.Any, *, require_api_key: bool = False, admin_key: str | None = None,
                 auth_manager=None, tool_parser: str | None = None, reasoning_parser: str | None = None,
                 tools: dict[str, tp.Callable] | None = None, response_store=None, default_max_tokens: int = 256,
                 storage_dir: str | None = None):
        from ....workers.auth import EnhancedApiKeyManager
        from ....workers.response_store import ResponseStore

        if not isinstance(engines, dict):
            engines = {getattr(engines, "name", None) or "default": engines}
        self.engines = engines
        self.auth = auth_manager or EnhancedApiKeyManager(require_api_key=require_api_key, admin_key=admin_key,
                                                          storage_dir=storage_dir)
        self.tool_parser_name, self.reasoning_parser_name = tool_parser, reasoning_parser
        self.tools = tools or {}
        self.tool_schemas: list[dict] = []
        self.store = response_store if response_store is not None else ResponseStore(None)
        self.default_max_tokens = default_max_tokens
        self.started = time.time()
        self.app = self._build()

    # ------------------------------------------------------------------ helpers
    def _engine(self, model: str | None):
        if model in self.engines:
            return model, self.engines[model]
        if model is None or len(self.engines) == 1:
            name = next(iter(self.engines))
            return name, self.engines[name]
        raise KeyError(model)

    def _parser(self, engine, want_tools: bool) -> DelegatingParser:
        mtype = getattr(getattr(engine, "model", None), "config", None)
        mtype = getattr(mtype, "model_type", None)
        tname = self.tool_parser_name or (detect_tool_parser(mtype, engine.tokenizer) if want_tools else None)
        rname = self.reasoning_parser_name or detect_reasoning_parser(mtype, engine.tokenizer)
        tp_ = ToolParserManager.get_tool_parser(tname)(engine.tokenizer) if (tname and want_tools) else None
        rp_ = ReasoningParserManager.get_reasoning_parser(rname)(engine.tokenizer) if rname else None
        return DelegatingParser(rp_, tp_)

    def register_tool(self, fn: tp.Callable, schema: dict | None = None) -> None:
        self.tools[fn.__name__] = fn
        self.tool_schemas.append(schema or {"type": "function", "function": {"name": fn.__name__,
                                                                               "description": fn.__doc__ or ""}})

    def _prompt_from_messages(self, engine, req: ChatCompletionRequest) -> str:
        msgs = [m.model_dump(exclude_none=True) for m in req.messages]
        tools = [t.model_dump(exclude_none=True) for t in req.tools] if req.tools else None
        return engine.tokenizer.apply_chat_template(msgs, tools=tools, tokenize=False,
                                                    add_generation_prompt=req.add_generation_prompt,
                                                    **(req.chat_template_kwargs or {}))

    # ------------------------------------------------------------------ app
    def _build(self):
        from ....workers.auth import AuthError

        app = FastAPI(title="eSurge API", version="1")
        server = self

        def key_of(request: Request) -> str | None:
            h = request.headers.get("authorization")
            if h and h.lower().startswith("bearer "):
                return h[7:].strip()
            return request.headers.get("x-api-key")

        def authorize(request: Request, endpoint: str, model=None, tokens=0, streaming=False, uses_tools=False):
            try:
                return server.auth.authorize(key_of(request), endpoint=endpoint, model=model,
                                             ip=request.client.host if request.client else None,
                                             requested_tokens=tokens, streaming=streaming, uses_tools=uses_tools)
            except AuthError as e:
                raise HTTPException(status_code=e.status_code, detail=str(e)) from e

        def need_admin(request: Request):
            if not server.auth.is_admin(key_of(request)):
                raise HTTPException(status_code=403, detail="admin key required")

        async def pump(request: Request, engine, iterator):
            """Moves a blocking engine iterator onto the event loop; stops it when the client goes away."""
            loop = asyncio.get_running_loop()
            it = iter(iterator)
            sentinel = object()
            try:
                while True:
                    item = await loop.run_in_executor(None, next, it, sentinel)
                    if item is sentinel:
                        return
                    if await request.is_disconnected():
                        return
                    yield item
            finally:
                close = getattr(it, "close", None)
                if close:
                    await loop.run_in_executor(None, close)

        @app.get("/health")
        async def health():
            return {"status": "ok", "uptime_s": time.time() - server.started,
                    "models": {n: {"running": e.num_running_requests, "waiting": e.num_pending_requests}
                               for n, e in server.engines.items()}}

        @app.get("/metrics")
        async def metrics():
            lines = []
            for name, e in server.engines.items():
                for k, v in e.get_metrics_summary().items():
                    if isinstance(v, (int, float)):
                        lines.append(f'esurge_{k}{{model="{name}"}} {v}')
            return PlainTextResponse("\n".join(lines) + "\n")

        @app.get("/v1/models")
        async def models(request: Request):
            authorize(request, "/v1/models")
            return ModelList(data=[ModelCard(id=n, max_model_len=e.max_model_len) for n, e in server.engines.items()])

        @app.get("/v1/models/{model_id}")
        async def model(model_id: str, request: Request):
            authorize(request, "/v1/models")
            if model_id not in server.engines:
                raise HTTPException(status_code=404, detail=f"model {model_id!r} not found")
            return ModelCard(id=model_id, max_model_len=server.engines[model_id].max_model_len)

        @app.post("/v1/chat/completions")
        async def chat(req: ChatCompletionRequest, request: Request):
            try:
                name, engine = server._engine(req.model)
            except KeyError:
                raise HTTPException(status_code=404, detail=f"model {req.model!r} not found") from None
            sp = req.to_sampling_params(server.default_max_tokens)
            rec = authorize(request, "/v1/chat/completions", name, sp.max_tokens or 0, req.stream, bool(req.tools))
            prompt = server._prompt_from_messages(engine, req)
            parser = server._parser(engine, bool(req.tools))
            if not req.stream:
                loop = asyncio.get_running_loop()
                out = (await loop.run_in_executor(None, engine.generate, prompt, sp))[0]
                parsed = parser.parse(out.get_text())
                calls = [ToolCall(**c) for c in parsed["tool_calls"]] or None
                server.auth.record_usage(rec, len(out.prompt_token_ids), out.num_generated_tokens)
                msg = ChatMessage(role="assistant", content=parsed["content"], tool_calls=calls,
                                  reasoning_content=parsed["reasoning_content"])
                return ChatCompletionResponse(model=name, usage=_usage(out), choices=[
                    ChatCompletionResponseChoice(message=msg, finish_reason=_finish_reason(out, bool(calls)))])

            async def gen():
                rid = None
                first = ChatCompletionStreamResponse(model=name, choices=[
                    ChatCompletionStreamResponseChoice(delta=DeltaMessage(role="assistant", content=""))])
                rid = first.id
                yield sse(first)
                last, text, any_tools = None, "", False
                async for out in pump(request, engine, engine.stream(prompt, sp)):
                    last = out
                    text += out.delta_text
                    d = parser.parse_streaming(text, final=out.finished)
                    any_tools = any_tools or bool(d["tool_calls"])
                    if d["content"] or d["reasoning_content"] or d["tool_calls"]:
                        delta = DeltaMessage(content=d["content"] or None,
                                             reasoning_content=d["reasoning_content"] or None,
                                             tool_calls=[ToolCall(**c) for c in d["tool_calls"]] or None)
                        yield sse(ChatCompletionStreamResponse(id=rid, model=name, choices=[
                            ChatCompletionStreamResponseChoice(delta=delta)]))
                if last is not None:
                    server.auth.record_usage(rec, len(last.prompt_token_ids), last.num_generated_tokens)
                    include_usage = bool((req.stream_options or {}).get("include_usage", True))
                    yield sse(ChatCompletionStreamResponse(id=rid, model=name, usage=_usage(last) if include_usage
                                                           else None, choices=[ChatCompletionStreamResponseChoice(
                                                               delta=DeltaMessage(),
                                                               finish_reason=_finish_reason(last, any_tools))]))
                yield sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")

        @app.post("/v1/completions")
        async def completions(req: CompletionRequest, request: Request):
            try:
                name, engine = server._engine(req.model)
            except KeyError:
                raise HTTPException(status_code=404, detail=f"model {req.model!r} not found") from None
            sp = req.to_sampling_params(server.default_max_tokens)
            rec = authorize(request, "/v1/completions", name, sp.max_tokens or 0, req.stream)
            prompts = req.prompt
            if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
                prompts = [prompts]
            if not req.stream:
                loop = asyncio.get_running_loop()
                outs = await loop.run_in_executor(None, engine.generate, list(prompts), sp)
                choices, usage = [], UsageInfo()
                for i, o in enumerate(outs):
                    text = ((o.prompt or "") if req.echo else "") + o.get_text()
                    choices.append(CompletionResponseChoice(index=i, text=text, finish_reason=_finish_reason(o, False)))
                    usage.prompt_tokens += len(o.prompt_token_ids)
                    usage.completion_tokens += o.num_generated_tokens
                usage.total_tokens = usage.prompt_tokens + usage.completion_tokens
                server.auth.record_usage(rec, usage.prompt_tokens, usage.completion_tokens)
                return CompletionResponse(model=name, choices=choices, usage=usage)

            async def gen():
                last = None
                cid = None
                async for out in pump(request, engine, engine.stream(prompts[0], sp)):
                    last = out
                    chunk = CompletionResponse(model=name, choices=[CompletionResponseChoice(
                        text=out.delta_text, finish_reason=_finish_reason(out, False) if out.finished else None)],
                        usage=_usage(out))
                    cid = cid or chunk.id
                    chunk.id = cid
                    yield sse(chunk)
                if last is not None:
                    server.auth.record_usage(rec, len(last.prompt_token_ids), last.num_generated_tokens)
                yield sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")

        @app.post("/v1/responses")
        async def responses(req: ResponsesRequest, request: Request):
            try:
                name, engine = server._engine(req.model)
            except KeyError:
                raise HTTPException(status_code=404, detail=f"model {req.model!r} not found") from None
            if req.max_output_tokens:
                req.max_tokens = req.max_output_tokens
            sp = req.to_sampling_params(server.default_max_tokens)
            rec = authorize(request, "/v1/responses", name, sp.max_tokens or 0, req.stream, bool(req.tools))
            history: list[dict] = []
            if req.previous_response_id:
                prev = server.store.get(req.previous_response_id)
                if prev is None:
                    raise HTTPException(status_code=404, detail="previous_response_id not found")
                history = list(prev["messages"])
            if req.instructions and not history:
                history.append({"role": "system", "content": req.instructions})
            if isinstance(req.input, str):
                history.append({"role": "user", "content": req.input})
            else:
                for item in req.input:
                    content = item.get("content")
                    if isinstance(content, list):
                        content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
                    history.append({"role": item.get("role", "user"), "content": content})
            prompt = engine.tokenizer.apply_chat_template(history, tokenize=False, add_generation_prompt=True)
            if req.stream:
                parser = server._parser(engine, bool(req.tools))
                builder = ResponsesStreamBuilder(model=name, previous_response_id=req.previous_response_id)

                async def gen():
                    for ev, payload in builder.start():
                        yield sse_frame(ev, payload)
                    last, text = None, ""
                    async for out in pump(request, engine, engine.stream(prompt, sp)):
                        last = out
                        text += out.delta_text
                        d = parser.parse_streaming(text, final=out.finished)
                        for ev, payload in builder.feed(d["reasoning_content"], d["content"], d["tool_calls"]):
                            yield sse_frame(ev, payload)
                    if last is None:      # the client went away before the first token
                        return
                    n_in, n_out = len(last.prompt_token_ids), last.num_generated_tokens
                    server.auth.record_usage(rec, n_in, n_out)
                    events, final = builder.finish({"input_tokens": n_in, "output_tokens": n_out,
                                                    "total_tokens": n_in + n_out})
                    if req.store:
                        server.store.put(final["id"], {"messages": history + [
                            {"role": "assistant", "content": final["output_text"]}]})
                    for ev, payload in events:
                        yield sse_frame(ev, payload)

                return StreamingResponse(gen(), media_type="text/event-stream")
            loop = asyncio.get_running_loop()
            out = (await loop.run_in_executor(None, engine.generate, prompt, sp))[0]
            parsed = server._parser(engine, bool(req.tools)).parse(out.get_text())
            server.auth.record_usage(rec, len(out.prompt_token_ids), out.num_generated_tokens)
            items: list[dict] = []
            if parsed["reasoning_content"]:
                items.append({"type": "reasoning", "summary": [{"type": "summary_text",
                                                                 "text": parsed["reasoning_content"]}]})
            for c in parsed["tool_calls"]:
                items.append({"type": "function_call", "call_id": c["id"], "name": c["function"]["name"],
                              "arguments": c["function"]["arguments"]})
            text = parsed["content"] or ""
            items.append({"type": "message", "role": "assistant", "status": "completed",
                          "content": [{"type": "output_text", "text": text, "annotations": []}]})
            resp = ResponsesResponse(model=name, output=items, output_text=text,
                                     previous_response_id=req.previous_response_id,
                                     usage={"input_tokens": len(out.prompt_token_ids),
                                            "output_tokens": out.num_generated_tokens,
                                            "total_tokens": len(out.prompt_token_ids) + out.num_generated_tokens})
            if req.store:
                server.store.put(resp.id, {"messages": history + [{"role": "assistant", "content": text}]})
            return resp

        @app.get("/v1/tools")
        async def list_tools(request: Request):
            authorize(request, "/v1/tools")
            return {"tools": server.tool_schemas, "parsers": ToolParserManager.names()}

        @app.post("/v1/tools/execute")
        async def execute_tool(req: ToolExecuteRequest, request: Request):
            authorize(request, "/v1/tools/execute", uses_tools=True)
            fn = server.tools.get(req.name)
            if fn is None:
                raise HTTPException(status_code=404, detail=f"tool {req.name!r} is not registered")
            try:
                res = fn(**req.arguments)
                if asyncio.iscoroutine(res):
                    res = await res
            except Exception as e:  # noqa: BLE001
                return JSONResponse({"name": req.name, "error": f"{type(e).__name__}: {e}"}, status_code=400)
            return {"name": req.name, "result": res}

        # ---- admin ---------------------------------------------------------------------------------------------
        @app.post("/v1/admin/keys")
        async def create_key(body: dict, request: Request):
            from ....workers.auth import Permissions, Quota, RateLimits

            need_admin(request)
            raw, rec = server.auth.generate_api_key(
                body.get("name", "key"), body.get("role", "user"), body.get("expires_in_days"),
                RateLimits(**body.get("rate_limits", {})), Quota(**body.get("quota", {})),
                Permissions(**body.get("permissions", {})), body.get("metadata"))
            return {"key": raw, **rec.public()}

        @app.get("/v1/admin/keys")
        async def list_keys(request: Request, role: str | None = None, status: str | None = None):
            need_admin(request)
            return {"keys": server.auth.list_keys(role, status)}

        @app.get("/v1/admin/keys/stats")
        async def key_stats(request: Request):
            need_admin(request)
            return server.auth.statistics()

        @app.get("/v1/admin/keys/{key_id}")
        async def get_key(key_id: str, request: Request):
            need_admin(request)
            rec = server.auth.get_key(key_id)
            if rec is None:
                raise HTTPException(status_code=404, detail="key not found")
            return rec.public()

        @app.patch("/v1/admin/keys/{key_id}")
        async def update_key(key_id: str, body: dict, request: Request):
            need_admin(request)
            rec = server.auth.update_key(key_id, **body)
            if rec is None:
                raise HTTPException(status_code=404, detail="key not found")
            return rec.public()

        @app.delete("/v1/admin/keys/{key_id}")
        async def delete_key(key_id: str, request: Request):
            need_admin(request)
            if not server.auth.delete_key(key_id):
                raise HTTPException(status_code=404, detail="key not found")
            return {"deleted": key_id}

        @app.post("/v1/admin/keys/{key_id}/{action}")
        async def key_action(key_id: str, action: str, request: Request):
            need_admin(request)
            fn = {"revoke": server.auth.revoke_key, "suspend": server.auth.suspend_key,
                  "reactivate": server.auth.reactivate_key}.get(action)
            if action == "rotate":
                raw = server.auth.rotate_key(key_id)
                if raw is None:
                    raise HTTPException(status_code=404, detail="key not found")
                return {"key": raw}
            if fn is None:
                raise HTTPException(status_code=400, detail=f"unknown action {action!r}")
            if not fn(key_id):
                raise HTTPException(status_code=404, detail="key not found")
            return {"key_id": key_id, "action": action}

        @app.get("/v1/admin/audit-logs")
        async def audit(request: Request, limit: int = 100, key_id: str | None = None, action: str | None = None):
            need_admin(request)
            return {"logs": server.auth.get_audit_logs(limit, key_id, action)}

        return app

    def run(self, host: str = "0.0.0.0", port: int = 8000, log_level: str = "info") -> None:
        import uvicorn

        for e in self.engines.values():
            e.initiate()
        uvicorn.run(self.app, host=host, port=port, log_level=log_level)

    fire = run


def create_app(engines, **kw):
    return eSurgeApiServer(engines, **kw).app
