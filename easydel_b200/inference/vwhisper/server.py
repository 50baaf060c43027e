"""OpenAI-compatible speech endpoints over :class:`vWhisperInference`
(easydel/inference/vwhisper/server.py:81-601): ``POST /v1/audio/transcriptions`` and ``/v1/audio/translations``
(multipart form: ``file``, ``language``, ``response_format`` = json | text | srt | verbose_json | vtt,
``timestamp_granularities``), ``GET /`` and ``/health``.
"""

from __future__ import annotations

import asyncio
import typing as tp
from enum import Enum

from fastapi import FastAPI, File, Form, HTTPException, UploadFile
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import PlainTextResponse
from pydantic import BaseModel, Field


class ResponseFormat(str, Enum):
    json = "json"
    text = "text"
    srt = "srt"
    verbose_json = "verbose_json"
    vtt = "vtt"


class TranscriptionResponse(BaseModel):
    text: str = Field(..., description="The transcribed text")
    segments: list[dict[str, tp.Any]] | None = Field(None, description="Segments with timestamps")


def _clock(t: float, sep: str) -> str:
    ms = int(round(t * 1000))
    h, ms = divmod(ms, 3600000)
    m, ms = divmod(ms, 60000)
    s, ms = divmod(ms, 1000)
    return f"{h:02d}:{m:02d}:{s:02d}{sep}{ms:03d}"


def to_srt(chunks) -> str:
    return "".join(f"{i}\n{_clock(c['timestamp'][0], ',')} --> {_clock(c['timestamp'][1], ',')}\n"
                   f"{(c['text'] or '').strip()}\n\n" for i, c in enumerate(chunks, 1))


def to_vtt(chunks) -> str:
    return "WEBVTT\n\n" + "".join(f"{_clock(c['timestamp'][0], '.')} --> {_clock(c['timestamp'][1], '.')}\n"
                                  f"{(c['text'] or '').strip()}\n\n" for c in chunks)


def create_whisper_app(inference, max_upload_bytes: int = 512 << 20) -> FastAPI:
    """``inference``: a :class:`vWhisperInference` (or any callable with its ``generate`` signature)."""
    app = FastAPI(title="easydel_b200 Whisper API", version="1.0.0")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])
    lock = asyncio.Lock()      # one utterance on the GPU at a time; windows of an utterance are batched inside

    @app.get("/")
    def root():
        return {"status": "ok", "endpoints": ["/v1/audio/transcriptions", "/v1/audio/translations"]}

    @app.get("/health")
    def health():
        return {"status": "healthy"}

    async def run(file: UploadFile, task: str, language, response_format: ResponseFormat, granularities):
        data = await file.read()
        if not data:
            raise HTTPException(400, "empty audio file")
        if len(data) > max_upload_bytes:
            raise HTTPException(413, "audio file too large")
        want_ts = response_format in (ResponseFormat.srt, ResponseFormat.vtt, ResponseFormat.verbose_json) or \
            bool(granularities)
        try:
            async with lock:
                out = await asyncio.get_running_loop().run_in_executor(
                    None, lambda: inference.generate(data, language=language, task=task, return_timestamps=want_ts))
        except (ValueError, RuntimeError) as e:
            raise HTTPException(400, str(e)) from e
        text = out.get("text") or ""
        chunks = out.get("chunks") or []
        if response_format == ResponseFormat.text:
            return PlainTextResponse(text)
        if response_format == ResponseFormat.srt:
            return PlainTextResponse(to_srt(chunks))
        if response_format == ResponseFormat.vtt:
            return PlainTextResponse(to_vtt(chunks), media_type="text/vtt")
        segs = [{"id": i, "start": c["timestamp"][0], "end": c["timestamp"][1], "text": c["text"]}
                for i, c in enumerate(chunks)] if want_ts else None
        if response_format == ResponseFormat.verbose_json:
            return {"task": task, "language": language, "duration": segs[-1]["end"] if segs else 0.0, "text": text,
                    "segments": segs}
        return TranscriptionResponse(text=text, segments=segs)

    @app.post("/v1/audio/transcriptions")
    async def transcriptions(file: UploadFile = File(...), model: str = Form("whisper"),
                             language: tp.Optional[str] = Form(None), prompt: tp.Optional[str] = Form(None),
                             response_format: ResponseFormat = Form(ResponseFormat.json),
                             temperature: float = Form(0.0),
                             timestamp_granularities: tp.Optional[str] = Form(None)):
        return await run(file, "transcribe", language, response_format, timestamp_granularities)

    @app.post("/v1/audio/translations")
    async def translations(file: UploadFile = File(...), model: str = Form("whisper"),
                           language: tp.Optional[str] = Form(None), prompt: tp.Optional[str] = Form(None),
                           response_format: ResponseFormat = Form(ResponseFormat.json),
                           temperature: float = Form(0.0)):
        return await run(file, "translate", language, response_format, None)

    return app


def run_server(inference, host: str = "0.0.0.0", port: int = 8000):
    import uvicorn

    uvicorn.run(create_whisper_app(inference), host=host, port=port)
