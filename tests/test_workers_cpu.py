"""Tokenizer / detokenizer worker processes over ZeroMQ, the Prometheus exporter and provisioning files."""

import torch

from easydel_b200.workers.pipeline import FastIncrementalDecoder, WorkerManager


class _Tok:
    eos_token_id = 2

    def __call__(self, text, add_special_tokens=True, **_):
        return {"input_ids": ([1] if add_special_tokens else []) + [ord(c) for c in text]}

    def decode(self, ids, skip_special_tokens=True):
        return bytes(i for i in ids if i > 2 and i < 256).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tools=None, tokenize=False, add_generation_prompt=True, **_):
        return "".join(f"<{m['role']}>{m['content']}" for m in messages) + ("<assistant>" if add_generation_prompt else "")


def _factory():
    return _Tok()


def test_incremental_decoder_holds_back_partial_utf8():
    d = FastIncrementalDecoder(_Tok())
    data = "héllo".encode()
    out = "".join(d.push([b]) for b in data)
    assert out == "héllo"


def test_worker_processes_roundtrip():
    with WorkerManager(_factory, startup_timeout=60) as mgr:
        tk, dk = mgr.client("tokenizer"), mgr.client("detokenizer")
        assert tk.call(op="ping")["kind"] == "tokenizer"
        ids = tk.tokenize("hi there")
        assert ids == [1] + [ord(c) for c in "hi there"]
        ids2 = tk.tokenize(messages=[{"role": "user", "content": "q"}])
        assert bytes(ids2[1:]).decode() == "<user>q<assistant>"
        text = "".join(dk.detokenize("r1", [t], finished=i == 2) for i, t in enumerate([104, 105, 33]))
        assert text == "hi!"
        tk.close()
        dk.close()


def test_prometheus_exporter_and_provisioning(tmp_path):
    from easydel_b200.inference.esurge import eSurge
    from easydel_b200.inference.esurge.monitoring import PrometheusMetrics, RichConsoleMonitor, eSurgeMonitoringServer
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128)
    eng = eSurge(LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32).eval(), max_model_len=128,
                 max_num_seqs=2, esurge_name="m")
    eng.generate([3, 4, 5], None)
    text = PrometheusMetrics(eng).render().decode()
    assert 'esurge_running_requests{model="m"}' in text and "esurge_kv_page_usage" in text
    assert "[m]" in RichConsoleMonitor(eng).line()
    files = eSurgeMonitoringServer(eng, prometheus_port=9191).write_provisioning(str(tmp_path))
    assert "esurge" in open(files["prometheus"]).read() and "panels" in open(files["grafana"]).read()


def test_distributed_controller_handshake_step_and_failure_detection():
    """Host-side failure detection: a wrong fingerprint, a diverging worker and a silent worker are all reported."""
    import socket

    import pytest

    from easydel_b200.inference.esurge.distributed import (DistributedController, WorkerControlServer, canonical_hash,
                                                           sampled_digest)

    def ep():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return f"tcp://127.0.0.1:{s.getsockname()[1]}"

    assert canonical_hash({"b": 1, "a": [1.0, 2]}) == canonical_hash({"a": [1.0, 2], "b": 1})
    e1, e2 = ep(), ep()
    good = WorkerControlServer(e1, "fp", step_fn=lambda d: {"r0": d["token"]}).start()
    bad = WorkerControlServer(e2, "fp", step_fn=lambda d: {"r0": d["token"] + 1}).start()
    try:
        ctl = DistributedController([e1], "fp", timeout_ms=2000)
        ctl.handshake()
        ctl.broadcast_step({"token": 7}, {"r0": 7})
        assert ctl.health()[0]["steps"] == 1
        with pytest.raises(RuntimeError, match="fingerprint"):
            DistributedController([e1], "other", timeout_ms=2000).handshake()
        with pytest.raises(RuntimeError, match="diverged"):
            DistributedController([e2], "fp", timeout_ms=2000).broadcast_step({"token": 7}, {"r0": 7})
        silent = DistributedController([ep()], "fp", timeout_ms=300)      # nobody listens there
        with pytest.raises(TimeoutError):
            silent.handshake()
        assert silent.health()[0]["ok"] is False
        assert sampled_digest({"a": 1}) != sampled_digest({"a": 2})
    finally:
        good.stop()
        bad.stop()
