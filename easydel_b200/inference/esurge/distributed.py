"""Multi-process control plane for eSurge (easydel/inference/esurge/distributed/*).

A serving job that spans several processes (tensor-parallel ranks on one box, or several boxes behind one
front end) needs every worker to run the same model with the same engine settings and to execute the same step
sequence. The leader (rank 0) owns the scheduler; before serving it checks every worker's *config fingerprint* (a
canonical hash of the engine settings and model config) and then drives them with small RPCs over ZeroMQ REQ/REP:
``hello`` (fingerprint exchange), ``step`` (a serialised scheduler decision; the worker answers with a digest of
the sampled tokens so that divergence is detected at once), ``health`` and ``shutdown``.

``DistributedController`` is the leader side, ``WorkerControlServer`` the worker side, ``WorkerRpcClient`` the
REQ socket with timeouts. Worker addresses come from a list or from DNS (``discover_workers``: all A records of a
service name, the usual layout of a headless Kubernetes service).
"""

from __future__ import annotations

import hashlib
import json
import socket
import threading
import time
import typing as tp


def canonical_hash(obj: tp.Any) -> str:
    """SHA-256 of a canonical JSON rendering (sorted keys, no whitespace, floats via repr)."""
    def norm(x):
        if isinstance(x, dict):
            return {str(k): norm(v) for k, v in sorted(x.items(), key=lambda kv: str(kv[0]))}
        if isinstance(x, (list, tuple)):
            return [norm(v) for v in x]
        if isinstance(x, float):
            return repr(x)
        if isinstance(x, (str, int, bool)) or x is None:
            return x
        return repr(x)

    return hashlib.sha256(json.dumps(norm(obj), separators=(",", ":")).encode()).hexdigest()


def config_fingerprint(engine) -> str:
    cfg = getattr(engine.model, "config", None)
    model_part = cfg.to_dict() if hasattr(cfg, "to_dict") else {}
    for k in ("_name_or_path", "transformers_version"):
        model_part.pop(k, None)
    return canonical_hash({"model": model_part, "max_model_len": engine.max_model_len,
                           "max_num_seqs": engine.max_num_seqs, "page_size": engine.page_size,
                           "max_num_batched_tokens": engine.max_num_batched_tokens})


def sampled_digest(sampled: dict[str, int]) -> str:
    return canonical_hash(sorted(sampled.items()))[:16]


def discover_workers(service: str, port: int) -> list[str]:
    """All addresses behind a DNS name -> ``tcp://ip:port`` endpoints (sorted, duplicates removed)."""
    infos = socket.getaddrinfo(service, port, proto=socket.IPPROTO_TCP)
    ips = sorted({i[4][0] for i in infos})
    return [f"tcp://{ip}:{port}" for ip in ips]


class WorkerRpcClient:
    def __init__(self, endpoint: str, timeout_ms: int = 10000):
        import zmq

        self.endpoint, self.timeout_ms = endpoint, timeout_ms
        self._ctx = zmq.Context.instance()
        self._sock = None

    def call(self, op: str, **payload) -> dict:
        import msgpack
        import zmq

        if self._sock is None:
            s = self._ctx.socket(zmq.REQ)
            for opt in (zmq.RCVTIMEO, zmq.SNDTIMEO):
                s.setsockopt(opt, self.timeout_ms)
            s.setsockopt(zmq.LINGER, 0)
            s.connect(self.endpoint)
            self._sock = s
        try:
            self._sock.send(msgpack.packb({"op": op, **payload}))
            return msgpack.unpackb(self._sock.recv(), raw=False)
        except zmq.Again as e:
            self._sock.close(0)
            self._sock = None
            raise TimeoutError(f"worker {self.endpoint} did not answer '{op}' within {self.timeout_ms} ms") from e

    def close(self):
        if self._sock is not None:
            self._sock.close(0)
            self._sock = None


class WorkerControlServer:
    """Runs next to a worker's engine; ``step_fn(decision) -> {request_id: token}`` executes one step."""

    def __init__(self, endpoint: str, fingerprint: str, step_fn: tp.Callable[[dict], dict[str, int]] | None = None):
        self.endpoint, self.fingerprint, self.step_fn = endpoint, fingerprint, step_fn
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        self.steps = 0

    def _loop(self, ready: threading.Event):
        import msgpack
        import zmq

        ctx = zmq.Context.instance()
        sock = ctx.socket(zmq.REP)
        sock.setsockopt(zmq.RCVTIMEO, 200)
        sock.setsockopt(zmq.LINGER, 0)
        sock.bind(self.endpoint)
        ready.set()
        while not self._stop.is_set():
            try:
                msg = msgpack.unpackb(sock.recv(), raw=False)
            except zmq.Again:
                continue
            op = msg.get("op")
            try:
                if op == "hello":
                    rep = {"ok": msg.get("fingerprint") == self.fingerprint, "fingerprint": self.fingerprint}
                elif op == "health":
                    rep = {"ok": True, "steps": self.steps, "time": time.time()}
                elif op == "step":
                    sampled = self.step_fn(msg["decision"]) if self.step_fn else {}
                    self.steps += 1
                    rep = {"ok": True, "digest": sampled_digest(sampled)}
                elif op == "shutdown":
                    rep = {"ok": True}
                    self._stop.set()
                else:
                    rep = {"ok": False, "error": f"unknown op {op!r}"}
            except Exception as e:  # noqa: BLE001
                rep = {"ok": False, "error": f"{type(e).__name__}: {e}"}
            sock.send(msgpack.packb(rep))
        sock.close(0)

    def start(self) -> "WorkerControlServer":
        ready = threading.Event()
        self._thread = threading.Thread(target=self._loop, args=(ready,), daemon=True)
        self._thread.start()
        ready.wait(10)
        return self

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)


class DistributedController:
    def __init__(self, endpoints: tp.Sequence[str], fingerprint: str, timeout_ms: int = 10000):
        self.clients = [WorkerRpcClient(e, timeout_ms) for e in endpoints]
        self.fingerprint = fingerprint

    def handshake(self) -> None:
        """Raises when a worker runs a different configuration or does not answer."""
        for c in self.clients:
            rep = c.call("hello", fingerprint=self.fingerprint)
            if not rep.get("ok"):
                raise RuntimeError(f"worker {c.endpoint} has fingerprint {rep.get('fingerprint')!r}, "
                                   f"leader has {self.fingerprint!r}")

    def broadcast_step(self, decision: dict, leader_sampled: dict[str, int]) -> None:
        want = sampled_digest(leader_sampled)
        for c in self.clients:
            rep = c.call("step", decision=decision)
            if not rep.get("ok"):
                raise RuntimeError(f"worker {c.endpoint} failed the step: {rep.get('error')}")
            if rep.get("digest") != want:
                raise RuntimeError(f"worker {c.endpoint} sampled different tokens (digest {rep.get('digest')} vs "
                                   f"{want}): the ranks have diverged")

    def health(self) -> list[dict]:
        out = []
        for c in self.clients:
            try:
                out.append({"endpoint": c.endpoint, **c.call("health")})
            except TimeoutError as e:
                out.append({"endpoint": c.endpoint, "ok": False, "error": str(e)})
        return out

    def shutdown(self) -> None:
        for c in self.clients:
            try:
                c.call("shutdown")
            except TimeoutError:
                pass
            c.close()
