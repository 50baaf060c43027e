"""Tokenizer / detokenizer worker processes with ZeroMQ endpoints
(easydel/workers/esurge/pipeline/worker_main.py:40-374, ``WorkerManager``).

Tokenisation of long prompts and incremental detokenisation of many streams are CPU work that would otherwise run
on the engine's scheduler thread. ``WorkerManager`` spawns one tokenizer and one detokenizer process bound to
``ipc://`` (or ``tcp://127.0.0.1``) endpoints; the clients speak msgpack over REQ/REP. The detokenizer keeps one
``FastIncrementalDecoder`` per request id so that only the new token ids travel.
"""

from __future__ import annotations

import multiprocessing as mp
import os
import tempfile
import time
import typing as tp
import uuid


class FastIncrementalDecoder:
    """Turns a growing token list into text deltas without re-decoding from the start and without emitting half
    of a multi-byte character."""

    def __init__(self, tokenizer, skip_special_tokens: bool = True, window: int = 6):
        self.tok, self.skip, self.window = tokenizer, skip_special_tokens, window
        self.ids: list[int] = []
        self.prefix_offset = self.read_offset = 0

    def push(self, new_ids: tp.Sequence[int]) -> str:
        self.ids.extend(int(t) for t in new_ids)
        prefix = self.tok.decode(self.ids[self.prefix_offset:self.read_offset], skip_special_tokens=self.skip)
        full = self.tok.decode(self.ids[self.prefix_offset:], skip_special_tokens=self.skip)
        if full.endswith("�") or len(full) <= len(prefix):
            return ""
        self.prefix_offset = max(self.read_offset - self.window, 0)
        self.read_offset = len(self.ids)
        return full[len(prefix):]


def _serve(endpoint: str, tokenizer_factory: tp.Callable[[], tp.Any], kind: str, ready) -> None:
    import msgpack
    import zmq

    tok = tokenizer_factory()
    ctx = zmq.Context()
    sock = ctx.socket(zmq.REP)
    sock.bind(endpoint)
    ready.set()
    decoders: dict[str, FastIncrementalDecoder] = {}
    while True:
        msg = msgpack.unpackb(sock.recv(), raw=False)
        op = msg.get("op")
        try:
            if op == "shutdown":
                sock.send(msgpack.packb({"ok": True}))
                break
            if op == "ping":
                rep = {"ok": True, "kind": kind, "pid": os.getpid()}
            elif op == "tokenize":
                if msg.get("messages") is not None:
                    text = tok.apply_chat_template(msg["messages"], tools=msg.get("tools"), tokenize=False,
                                                   add_generation_prompt=msg.get("add_generation_prompt", True))
                else:
                    text = msg["text"]
                ids = tok(text, add_special_tokens=msg.get("add_special_tokens", True))["input_ids"]
                rep = {"ok": True, "input_ids": list(ids), "text": text}
            elif op == "detokenize":
                rid = msg["request_id"]
                d = decoders.get(rid)
                if d is None:
                    d = decoders[rid] = FastIncrementalDecoder(tok, msg.get("skip_special_tokens", True))
                delta = d.push(msg["token_ids"])
                if msg.get("finished"):
                    decoders.pop(rid, None)
                rep = {"ok": True, "delta": delta}
            elif op == "reset":
                decoders.pop(msg["request_id"], None)
                rep = {"ok": True}
            else:
                rep = {"ok": False, "error": f"unknown op {op!r}"}
        except Exception as e:  # noqa: BLE001
            rep = {"ok": False, "error": f"{type(e).__name__}: {e}"}
        sock.send(msgpack.packb(rep))
    sock.close(0)
    ctx.term()


class WorkerClient:
    def __init__(self, endpoint: str, timeout_ms: int = 30000):
        import zmq

        self.endpoint, self.timeout_ms = endpoint, timeout_ms
        self._ctx = zmq.Context.instance()
        self._sock = None

    def _socket(self):
        import zmq

        if self._sock is None:
            s = self._ctx.socket(zmq.REQ)
            s.setsockopt(zmq.RCVTIMEO, self.timeout_ms)
            s.setsockopt(zmq.SNDTIMEO, self.timeout_ms)
            s.setsockopt(zmq.LINGER, 0)
            s.connect(self.endpoint)
            self._sock = s
        return self._sock

    def call(self, **msg) -> dict:
        import msgpack
        import zmq

        s = self._socket()
        try:
            s.send(msgpack.packb(msg))
            rep = msgpack.unpackb(s.recv(), raw=False)
        except zmq.Again as e:
            self._sock.close(0)
            self._sock = None      # a REQ socket that missed its reply cannot be reused
            raise TimeoutError(f"worker at {self.endpoint} did not answer within {self.timeout_ms} ms") from e
        if not rep.get("ok"):
            raise RuntimeError(rep.get("error", "worker error"))
        return rep

    def tokenize(self, text: str | None = None, messages=None, **kw) -> list[int]:
        return self.call(op="tokenize", text=text, messages=messages, **kw)["input_ids"]

    def detokenize(self, request_id: str, token_ids: tp.Sequence[int], finished: bool = False, **kw) -> str:
        return self.call(op="detokenize", request_id=request_id, token_ids=list(token_ids), finished=finished,
                         **kw)["delta"]

    def close(self):
        if self._sock is not None:
            self._sock.close(0)
            self._sock = None


class WorkerManager:
    """Spawns the tokenizer and detokenizer processes and hands out clients; ``startup_timeout`` bounds the wait."""

    def __init__(self, tokenizer_factory: tp.Callable[[], tp.Any], startup_timeout: float = 60.0,
                 transport: str = "ipc"):
        self.factory, self.startup_timeout, self.transport = tokenizer_factory, startup_timeout, transport
        self.procs: dict[str, mp.Process] = {}
        self.endpoints: dict[str, str] = {}
        self._dir = tempfile.mkdtemp(prefix="edl-workers-")

    def _endpoint(self, kind: str) -> str:
        if self.transport == "ipc":
            return f"ipc://{self._dir}/{kind}-{uuid.uuid4().hex[:8]}"
        import socket

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return f"tcp://127.0.0.1:{s.getsockname()[1]}"

    def start(self) -> "WorkerManager":
        ctx = mp.get_context("spawn")
        for kind in ("tokenizer", "detokenizer"):
            ep = self._endpoint(kind)
            ready = ctx.Event()
            p = ctx.Process(target=_serve, args=(ep, self.factory, kind, ready), daemon=True)
            p.start()
            if not ready.wait(self.startup_timeout):
                p.terminate()
                raise TimeoutError(f"{kind} worker did not start within {self.startup_timeout}s")
            self.procs[kind], self.endpoints[kind] = p, ep
        return self

    def client(self, kind: str, timeout_ms: int = 30000) -> WorkerClient:
        return WorkerClient(self.endpoints[kind], timeout_ms)

    def stop(self) -> None:
        for kind, p in self.procs.items():
            try:
                WorkerClient(self.endpoints[kind], 2000).call(op="shutdown")
            except Exception:  # noqa: BLE001
                pass
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
        self.procs.clear()

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
