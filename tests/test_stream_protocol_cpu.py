"""The Responses API event stream: event order, indices and sequence numbers, the final object, and the endpoint."""

import json

import pytest

from easydel_b200.inference.stream_protocol import ResponsesStreamBuilder, sse_frame, stream_delta


def test_stream_delta_rules():
    assert stream_delta("hello world", "hello") == " world"
    assert stream_delta("hello", "hello") == ""
    assert stream_delta("", "") == ""
    # the parser rewrote the start of the text: send what follows the longest overlap with what was sent
    assert stream_delta("lo world", "hello") == " world"
    # nothing in common: the engine's own delta, unless it went out already
    assert stream_delta("abc", "xyz", "c") == "c"
    assert stream_delta("abc", "xyz", "z") == ""
    assert stream_delta("abc", "xyz") == ""
    assert stream_delta("abc", None) == "abc"


def test_sse_frame_layout():
    assert sse_frame("response.created", {"a": 1}) == 'event: response.created\ndata: {"a":1}\n\n'
    assert sse_frame(None, "[DONE]") == "data: [DONE]\n\n"
    assert json.loads(sse_frame("e", {"t": "é"}).split("data: ")[1]) == {"t": "é"}


def _names(events):
    return [n for n, _ in events]


def test_reasoning_then_tool_call_then_message():
    b = ResponsesStreamBuilder(model="m", response_id="resp_1", created_at=7)
    ev = b.start()
    assert _names(ev) == ["response.created", "response.in_progress"]
    assert ev[0][1]["response"]["status"] == "in_progress" and ev[0][1]["response"]["output"] == []
    ev += b.feed(reasoning_delta="think ")
    ev += b.feed(reasoning_delta="hard")
    call = {"id": "call_9", "type": "function", "function": {"name": "f", "arguments": '{"a": 1}'}}
    ev += b.feed(tool_calls=[call])
    ev += b.feed(content_delta="Done")
    ev += b.feed(content_delta=".")
    tail, final = b.finish({"input_tokens": 5, "output_tokens": 9, "total_tokens": 14})
    ev += tail
    assert _names(ev) == [
        "response.created", "response.in_progress",
        "response.output_item.added", "response.reasoning_summary_part.added",
        "response.reasoning_summary_text.delta", "response.reasoning_summary_text.delta",
        "response.reasoning_summary_text.done", "response.reasoning_summary_part.done", "response.output_item.done",
        "response.output_item.added", "response.function_call_arguments.delta",
        "response.function_call_arguments.done", "response.output_item.done",
        "response.output_item.added", "response.content_part.added",
        "response.output_text.delta", "response.output_text.delta",
        "response.output_text.done", "response.content_part.done", "response.output_item.done",
        "response.completed"]
    assert [p["sequence_number"] for _, p in ev] == list(range(len(ev)))
    assert all(p["type"] == n for n, p in ev)
    added = [p for n, p in ev if n == "response.output_item.added"]
    assert [p["output_index"] for p in added] == [0, 1, 2]
    assert [p["item"]["type"] for p in added] == ["reasoning", "function_call", "message"]
    # deltas point at the item that was opened for them
    deltas = [p for n, p in ev if n == "response.output_text.delta"]
    assert {p["item_id"] for p in deltas} == {added[2]["item"]["id"]} and "".join(p["delta"] for p in deltas) == "Done."
    assert final["status"] == "completed" and final["output_text"] == "Done." and final["usage"]["total_tokens"] == 14
    kinds = [it["type"] for it in final["output"]]
    assert kinds == ["reasoning", "function_call", "message"]
    assert final["output"][0]["summary"] == [{"type": "summary_text", "text": "think hard"}]
    assert final["output"][1]["call_id"] == "call_9" and json.loads(final["output"][1]["arguments"]) == {"a": 1}
    assert final["output"][2]["content"][0]["text"] == "Done." and all(it["status"] == "completed"
                                                                       for it in final["output"])
    assert ev[-1][1]["response"] == final and final["id"] == "resp_1" and final["created_at"] == 7
    with pytest.raises(RuntimeError):
        b.feed(content_delta="late")
    with pytest.raises(RuntimeError):
        b.finish()


def test_empty_generation_still_carries_a_message():
    b = ResponsesStreamBuilder(model="m")
    b.start()
    events, final = b.finish()
    assert [it["type"] for it in final["output"]] == ["message"] and final["output_text"] == ""
    assert _names(events)[-1] == "response.completed" and final["usage"] is None


def test_two_tool_calls_and_dict_arguments():
    b = ResponsesStreamBuilder(model="m")
    b.start()
    ev = b.feed(tool_calls=[{"function": {"name": "f", "arguments": {"a": 1}}}])
    ev += b.feed(content_delta="\n")                   # white space between calls opens nothing
    ev += b.feed(tool_calls=[{"function": {"name": "g", "arguments": "{}"}}])
    _, final = b.finish()
    assert [it["type"] for it in final["output"]] == ["function_call", "function_call"]
    assert final["output"][0]["arguments"] == '{"a":1}' and final["output"][0]["call_id"].startswith("call_")
    assert "response.output_text.delta" not in _names(ev)


def _frames(body: str):
    out = []
    for block in body.strip().split("\n\n"):
        lines = dict(line.split(": ", 1) for line in block.split("\n"))
        out.append((lines.get("event"), json.loads(lines["data"])))
    return out


def test_responses_endpoint_streams_typed_events(tmp_path):
    from starlette.testclient import TestClient

    from easydel_b200.inference.esurge.server import eSurgeApiServer
    from easydel_b200.workers.response_store import ResponseStore
    from test_api_server_cpu import make_engine

    client = TestClient(eSurgeApiServer(make_engine(), response_store=ResponseStore(str(tmp_path))).app)
    body = {"input": "first", "max_output_tokens": 4, "temperature": 0, "ignore_eos": True}
    plain = client.post("/v1/responses", json=body).json()
    with client.stream("POST", "/v1/responses", json=dict(body, stream=True)) as r:
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        frames = _frames("".join(r.iter_text()))
    names = [n for n, _ in frames]
    assert names[:2] == ["response.created", "response.in_progress"] and names[-1] == "response.completed"
    assert all(p["type"] == n for n, p in frames)
    assert [p["sequence_number"] for _, p in frames] == list(range(len(frames)))
    final = frames[-1][1]["response"]
    text = "".join(p["delta"] for n, p in frames if n == "response.output_text.delta")
    assert text == final["output_text"] == plain["output_text"]
    assert final["usage"]["output_tokens"] == 4 and final["usage"]["input_tokens"] == plain["usage"]["input_tokens"]
    # the streamed response was stored and can be continued
    nxt = client.post("/v1/responses", json=dict(body, input="second", previous_response_id=final["id"])).json()
    assert nxt["previous_response_id"] == final["id"] and nxt["usage"]["input_tokens"] > final["usage"]["input_tokens"]
