"""OpenAI-compatible server over a tiny CPU engine: completions, chat (plain + SSE), responses with
``previous_response_id``, tools, auth (keys, rate limits, admin endpoints) and the parsers."""

import json

import pytest
import torch
from starlette.testclient import TestClient

from easydel_b200.inference.esurge import eSurge
from easydel_b200.inference.esurge.server import eSurgeApiServer
from easydel_b200.inference.reasoning import ReasoningParserManager
from easydel_b200.inference.tools import ToolParserManager
from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
from easydel_b200.workers.auth import AuthError, EnhancedApiKeyManager, Permissions, RateLimits
from easydel_b200.workers.response_store import ResponseStore

V = 128


class Tok:
    pad_token_id, bos_token_id, eos_token_id = 0, 1, 2

    def __call__(self, text, add_special_tokens=True, **_):
        return {"input_ids": ([1] if add_special_tokens else []) + [3 + (ord(c) % (V - 3)) for c in text]}

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(32 + ((i - 3) % 95)) for i in ids if i >= 3)

    def apply_chat_template(self, messages, tools=None, tokenize=False, add_generation_prompt=True, **_):
        s = "".join(f"<{m['role']}>{m.get('content') or ''}" for m in messages)
        return s + ("<assistant>" if add_generation_prompt else "")

    def get_vocab(self):
        return {}


def make_engine():
    cfg = LlamaConfig(vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=512, eos_token_id=2)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    return eSurge(model, tokenizer=Tok(), max_model_len=256, max_num_seqs=4, esurge_name="tiny")


@pytest.fixture(scope="module")
def engine():
    return make_engine()


def test_completions_and_chat(engine):
    client = TestClient(eSurgeApiServer(engine).app)
    assert client.get("/health").json()["status"] == "ok"
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    assert client.get("/v1/models/nope").status_code == 404
    r = client.post("/v1/completions", json={"model": "tiny", "prompt": "hello", "max_tokens": 5, "temperature": 0,
                                             "ignore_eos": True})
    body = r.json()
    assert r.status_code == 200 and body["usage"]["completion_tokens"] == 5 and body["choices"][0]["text"]
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                  "temperature": 0, "ignore_eos": True})
    body = r.json()
    assert body["choices"][0]["message"]["role"] == "assistant" and body["usage"]["completion_tokens"] == 4
    greedy_text = body["choices"][0]["message"]["content"]
    # SSE stream carries the same text
    with client.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                             "max_tokens": 4, "temperature": 0, "ignore_eos": True,
                                                             "stream": True}) as s:
        frames = [l[6:] for l in s.iter_lines() if l.startswith("data: ")]
    assert frames[-1] == "[DONE]"
    chunks = [json.loads(f) for f in frames[:-1]]
    text = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks)
    assert text == greedy_text and chunks[-1]["choices"][0]["finish_reason"] == "length"
    assert "esurge_" in client.get("/metrics").text


def test_responses_api_threads_conversations(engine, tmp_path):
    srv = eSurgeApiServer(engine, response_store=ResponseStore(str(tmp_path)))
    client = TestClient(srv.app)
    r1 = client.post("/v1/responses", json={"input": "first", "max_output_tokens": 3, "temperature": 0,
                                            "ignore_eos": True}).json()
    assert r1["object"] == "response" and r1["usage"]["output_tokens"] == 3
    r2 = client.post("/v1/responses", json={"input": "second", "previous_response_id": r1["id"],
                                            "max_output_tokens": 3, "temperature": 0, "ignore_eos": True}).json()
    assert r2["previous_response_id"] == r1["id"] and r2["usage"]["input_tokens"] > r1["usage"]["input_tokens"]
    assert client.post("/v1/responses", json={"input": "x", "previous_response_id": "resp-missing"}).status_code == 404
    assert len(ResponseStore(str(tmp_path))) == 2    # persisted


def test_tools_endpoints(engine):
    srv = eSurgeApiServer(engine)

    def add(a: int, b: int):
        """adds"""
        return a + b

    srv.register_tool(add)
    client = TestClient(srv.app)
    assert client.get("/v1/tools").json()["tools"][0]["function"]["name"] == "add"
    assert client.post("/v1/tools/execute", json={"name": "add", "arguments": {"a": 2, "b": 3}}).json()["result"] == 5
    assert client.post("/v1/tools/execute", json={"name": "nope"}).status_code == 404
    assert client.post("/v1/tools/execute", json={"name": "add", "arguments": {"a": 1}}).status_code == 400


def test_auth_flow(engine, tmp_path):
    srv = eSurgeApiServer(engine, require_api_key=True, admin_key="root-key", storage_dir=str(tmp_path))
    client = TestClient(srv.app)
    body = {"prompt": "x", "max_tokens": 2, "temperature": 0, "ignore_eos": True}
    assert client.post("/v1/completions", json=body).status_code == 401
    assert client.post("/v1/admin/keys", json={"name": "k"}).status_code == 403
    admin = {"Authorization": "Bearer root-key"}
    created = client.post("/v1/admin/keys", headers=admin,
                          json={"name": "k", "rate_limits": {"requests_per_minute": 2}}).json()
    hdr = {"Authorization": "Bearer " + created["key"]}
    assert client.post("/v1/completions", json=body, headers=hdr).status_code == 200
    assert client.post("/v1/completions", json=body, headers=hdr).status_code == 200
    assert client.post("/v1/completions", json=body, headers=hdr).status_code == 429
    kid = created["key_id"]
    assert client.get(f"/v1/admin/keys/{kid}", headers=admin).json()["total_completion_tokens"] == 4
    assert client.post(f"/v1/admin/keys/{kid}/suspend", headers=admin).status_code == 200
    assert client.post("/v1/completions", json=body, headers=hdr).status_code == 403
    new = client.post(f"/v1/admin/keys/{kid}/rotate", headers=admin).json()["key"]
    assert new != created["key"]
    logs = client.get("/v1/admin/audit-logs", headers=admin).json()["logs"]
    assert {"create", "suspend", "rotate"} <= {l["action"] for l in logs}
    # persisted store reloads
    again = EnhancedApiKeyManager(require_api_key=True, storage_dir=str(tmp_path))
    assert again.get_key(kid) is not None and again.get_key(kid).status == "suspended"


def test_key_permissions():
    m = EnhancedApiKeyManager(require_api_key=True)
    raw, rec = m.generate_api_key("p", permissions=Permissions(allowed_models=["tiny*"], allowed_ips=["10.*"],
                                                                 max_tokens_per_request=8, enable_streaming=False))
    assert m.authorize(raw, endpoint="/v1/completions", model="tiny-1", ip="10.0.0.1", requested_tokens=4) is rec
    for kw in (dict(model="big"), dict(ip="1.2.3.4"), dict(requested_tokens=9), dict(streaming=True)):
        args = dict(endpoint="/v1/completions", model="tiny-1", ip="10.0.0.1", requested_tokens=4)
        args.update(kw)
        with pytest.raises(AuthError) as e:
            m.authorize(raw, **args)
        assert e.value.status_code == 403
    raw2, _ = m.generate_api_key("r", rate_limits=RateLimits(tokens_per_minute=10))
    rec2 = m.authorize(raw2, endpoint="/v1/completions")
    m.record_usage(rec2, 6, 6)
    with pytest.raises(AuthError) as e:
        m.authorize(raw2, endpoint="/v1/completions")
    assert e.value.status_code == 429


CASES = {
    "hermes": 'ok <tool_call>\n{"name": "f", "arguments": {"a": 1}}\n</tool_call>',
    "llama3_json": '<|python_tag|>{"name": "f", "parameters": {"a": 1}}',
    "mistral": '[TOOL_CALLS][{"name": "f", "arguments": {"a": 1}}]',
    "pythonic": "[f(a=1)]",
    "qwen3_coder": "<tool_call>\n<function=f>\n<parameter=a>\n1\n</parameter>\n</function>\n</tool_call>",
    "glm45": "<tool_call>f\n<arg_key>a</arg_key>\n<arg_value>1</arg_value>\n</tool_call>",
    "deepseek_v3": "<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>f\n```json\n{\"a\": 1}\n```"
                   "<｜tool▁call▁end｜><｜tool▁calls▁end｜>",
    "deepseek_v31": '<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>f<｜tool▁sep｜>{"a": 1}<｜tool▁call▁end｜>',
    "kimi_k2": '<|tool_calls_section_begin|><|tool_call_begin|>functions.f:0<|tool_call_argument_begin|>{"a":1}'
               "<|tool_call_end|><|tool_calls_section_end|>",
    "openai": '<|channel|>commentary to=functions.f <|constrain|>json<|message|>{"a":1}<|call|>',
    "minimax_m2": '<minimax:tool_call><invoke name="f"><parameter name="a">1</parameter></invoke></minimax:tool_call>',
    "seed_oss": "<seed:tool_call><function=f><parameter=a>1</parameter></function></seed:tool_call>",
    "granite": '<|tool_call|>[{"name": "f", "arguments": {"a": 1}}]',
    "internlm": '<|action_start|><|plugin|>\n{"name": "f", "parameters": {"a": 1}}<|action_end|>',
    "jamba": '<tool_calls>[{"name": "f", "arguments": {"a": 1}}]</tool_calls>',
    "phi4_mini_json": 'functools[{"name": "f", "arguments": {"a": 1}}]',
    "xlam": '```json\n[{"name": "f", "arguments": {"a": 1}}]\n```',
    "olmo3": "<function_calls>f(a=1)</function_calls>",
    "functiongemma": "<start_function_call>call:f{a:1}<end_function_call>",
    "step3": '<｜tool_calls_begin｜><｜tool_call_begin｜>function<｜tool_sep｜><steptml:invoke name="f">'
             '<steptml:parameter name="a">1</steptml:parameter></steptml:invoke><｜tool_call_end｜><｜tool_calls_end｜>',
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_tool_parsers(name):
    res = ToolParserManager.get_tool_parser(name)(None).extract_tool_calls(CASES[name])
    assert res.tools_called, name
    fn = res.tool_calls[0]["function"]
    assert fn["name"] == "f" and json.loads(fn["arguments"]) == {"a": 1}
    plain = ToolParserManager.get_tool_parser(name)(None).extract_tool_calls("just words")
    assert not plain.tools_called and plain.content == "just words"


def test_all_registered_parsers_construct():
    for n in ToolParserManager.names():
        assert not ToolParserManager.get_tool_parser(n)(None).extract_tool_calls("no calls here.").tools_called
    assert len(ToolParserManager.names()) >= 33
    for n in ReasoningParserManager.names():
        ReasoningParserManager.get_reasoning_parser(n)(None).extract_reasoning("text")
    assert len(ReasoningParserManager.names()) >= 15


def test_reasoning_streaming_matches_offline():
    text = "<think>\nstep one\nstep two\n</think>\n\nfinal answer"
    p = ReasoningParserManager.get_reasoning_parser("qwen3")(None)
    r_all, c_all = "", ""
    for i in range(1, len(text) + 1):
        dr, dc = p.extract_reasoning_streaming(text[:i], final=i == len(text))
        r_all += dr
        c_all += dc
    off = ReasoningParserManager.get_reasoning_parser("qwen3")(None).extract_reasoning(text)
    assert r_all.strip("\n") == off[0] and c_all.strip("\n") == off[1]
