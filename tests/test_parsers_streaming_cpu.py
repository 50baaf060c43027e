"""Streaming behaviour of the tool-call and reasoning parsers: what has been sent stays sent, markers never leak
into content, calls are reported once and in order, and the streamed pieces add up to the offline result."""

import json

import pytest

from easydel_b200.inference.reasoning import (DelegatingParser, ReasoningParserManager, detect_reasoning_parser)
from easydel_b200.inference.tools.parsers import ToolParserManager
from test_api_server_cpu import CASES


def _stream_tools(parser, text, step):
    content, calls, when = "", [], []
    for i in range(step, len(text) + step, step):
        i = min(i, len(text))
        d, c = parser.extract_tool_calls_streaming(text[:i], final=i == len(text))
        content += d
        calls += c
        when += [i] * len(c)
    return content, calls, when


def _stream_reasoning(parser, text, step=1):
    r = c = ""
    for i in range(step, len(text) + step, step):
        i = min(i, len(text))
        dr, dc = parser.extract_reasoning_streaming(text[:i], final=i == len(text))
        r += dr
        c += dc
    return r, c


@pytest.mark.parametrize("step", [1, 5, 10_000])
@pytest.mark.parametrize("name", sorted(CASES))
def test_every_tool_parser_streams_its_call(name, step):
    lead = "" if name in ("pythonic", "llama3_json") else "Sure. "
    text = lead + CASES[name]
    content, calls, _ = _stream_tools(ToolParserManager.get_tool_parser(name)(None), text, step)
    assert len(calls) == 1 and calls[0]["index"] == 0
    fn = calls[0]["function"]
    assert fn["name"] == "f" and json.loads(fn["arguments"]) == {"a": 1}
    off = ToolParserManager.get_tool_parser(name)(None).extract_tool_calls(text)
    assert content.strip() == (off.content or "").strip() or content.strip() == lead.strip()
    assert "<" not in content and "[" not in content          # no marker fragment reaches the client


def test_hermes_two_calls_in_order_and_first_before_the_end():
    text = ('Let me check. <tool_call>\n{"name": "f", "arguments": {"a": 1}}\n</tool_call>\n'
            '<tool_call>\n{"name": "g", "arguments": {"b": "x"}}\n</tool_call>')
    content, calls, when = _stream_tools(ToolParserManager.get_tool_parser("hermes")(None), text, 1)
    assert content == "Let me check. "
    assert [(c["index"], c["function"]["name"]) for c in calls] == [(0, "f"), (1, "g")]
    assert json.loads(calls[1]["function"]["arguments"]) == {"b": "x"}
    assert when[0] < len(text) and when[1] == len(text)        # the first call goes out while the second grows
    assert len({c["id"] for c in calls}) == 2


def test_plain_text_with_marker_lookalikes_streams_through():
    text = "a < b and <tool is not a call"
    p = ToolParserManager.get_tool_parser("hermes")(None)
    seen = ""
    for i in range(1, len(text) + 1):
        d, calls = p.extract_tool_calls_streaming(text[:i], final=i == len(text))
        assert not calls
        seen += d
        assert text.startswith(seen)
    assert seen == text


def test_partial_marker_is_held_back_until_resolved():
    p = ToolParserManager.get_tool_parser("hermes")(None)
    d, _ = p.extract_tool_calls_streaming("ok <tool_c")
    assert d == "ok "
    d, _ = p.extract_tool_calls_streaming("ok <tool_cabinet")         # it was not a marker after all
    assert d == "<tool_cabinet"
    p = ToolParserManager.get_tool_parser("hermes")(None)
    d, _ = p.extract_tool_calls_streaming("ok <tool_c", final=True)    # the end of the stream flushes it
    assert d == "ok <tool_c"


def test_malformed_and_unterminated_calls():
    hermes = ToolParserManager.get_tool_parser("hermes")
    bad = '<tool_call>\n{"name": "f", "arguments": {"a": \n</tool_call>'
    res = hermes(None).extract_tool_calls(bad)
    assert not res.tools_called and res.content == bad
    open_ended = 'x <tool_call>\n{"name": "f", "arguments": {"a": 1}}'
    res = hermes(None).extract_tool_calls(open_ended)
    assert res.tools_called and res.content == "x" and json.loads(res.tool_calls[0]["function"]["arguments"]) == {"a": 1}


def test_multiple_calls_offline():
    res = ToolParserManager.get_tool_parser("mistral")(None).extract_tool_calls(
        '[TOOL_CALLS][{"name": "f", "arguments": {"a": 1}}, {"name": "g", "arguments": {}}]')
    assert [c["function"]["name"] for c in res.tool_calls] == ["f", "g"]
    res = ToolParserManager.get_tool_parser("pythonic")(None).extract_tool_calls(
        '[f(a=1, b="s", c=[1,2], d={"k": None}), g()]')
    assert json.loads(res.tool_calls[0]["function"]["arguments"]) == {"a": 1, "b": "s", "c": [1, 2], "d": {"k": None}}
    assert res.tool_calls[1]["function"] == {"name": "g", "arguments": "{}"}
    res = ToolParserManager.get_tool_parser("llama3_json")(None).extract_tool_calls(
        '{"name": "f", "parameters": {"a": 1}}; {"name": "g", "parameters": {}}')
    assert [c["function"]["name"] for c in res.tool_calls] == ["f", "g"]


def test_harmony_tool_stream_hides_channel_markup():
    text = ('<|channel|>analysis<|message|>need two tools<|end|><|start|>assistant<|channel|>commentary '
            'to=functions.f <|constrain|>json<|message|>{"a":1}<|call|><|start|>assistant<|channel|>commentary '
            'to=functions.g <|constrain|>json<|message|>{"b": 2}<|call|><|start|>assistant<|channel|>final'
            '<|message|>Done now.<|return|>')
    for step in (1, 4, 10_000):
        content, calls, when = _stream_tools(ToolParserManager.get_tool_parser("openai")(None), text, step)
        assert content == "Done now."
        assert [(c["index"], c["function"]["name"], json.loads(c["function"]["arguments"])) for c in calls] == [
            (0, "f", {"a": 1}), (1, "g", {"b": 2})]
        if step == 1:
            assert when[0] < when[1] < len(text)                # each call goes out at its own closing marker
    off = ToolParserManager.get_tool_parser("openai")(None).extract_tool_calls(text)
    assert off.content == "Done now." and len(off.tool_calls) == 2


def test_unknown_parser_names_raise():
    with pytest.raises(KeyError):
        ToolParserManager.get_tool_parser("no-such-parser")
    with pytest.raises(KeyError):
        ReasoningParserManager.get_reasoning_parser("no-such-parser")


REASONING = {
    "deepseek_r1": "thinking\nhard</think>\n\nanswer",
    "qwen3": "<think>\nthinking\nhard\n</think>\n\nanswer",
    "qwen3_thinking": "thinking\nhard\n</think>\n\nanswer",
    "ernie45": "thinking\nhard</think>\n<response>answer</response>",
    "hunyuan_a13b": "<think>\nthinking\nhard\n</think>\n<answer>\nanswer\n</answer>",
    "granite": "Here is my thought process:thinking\nhard\nHere is my response:answer",
    "mistral": "[THINK]thinking\nhard[/THINK]answer",
    "seed_oss": "<seed:think>thinking\nhard</seed:think>answer",
    "gemma4": "<|channel>thought\nthinking\nhard<channel|>answer",
    "gpt_oss": "<|channel|>analysis<|message|>thinking\nhard<|end|><|start|>assistant<|channel|>final<|message|>"
               "answer<|return|>",
    "glm45": "<think>thinking\nhard</think>\nanswer",
    "identity": "answer",
}


@pytest.mark.parametrize("step", [1, 3, 10_000])
@pytest.mark.parametrize("name", sorted(REASONING))
def test_reasoning_stream_adds_up_to_offline(name, step):
    text = REASONING[name]
    make = ReasoningParserManager.get_reasoning_parser(name)
    r_off, c_off = make(None).extract_reasoning(text)
    assert c_off == "answer"
    assert r_off == (None if name == "identity" else "thinking\nhard")
    r, c = _stream_reasoning(make(None), text, step)
    assert r.strip("\n") == (r_off or "") and c.strip("\n") == c_off
    for frag in ("think>", "<|", "|>", "<response", "<answer", "[THINK", "[/THINK", "Here is my"):
        assert frag not in r and frag not in c


def test_reasoning_without_end_marker():
    qwen = ReasoningParserManager.get_reasoning_parser("qwen3")(None)
    assert qwen.extract_reasoning("just an answer") == (None, "just an answer")
    assert qwen.extract_reasoning("<think>never closed") == ("never closed", None)
    r1 = ReasoningParserManager.get_reasoning_parser("deepseek_r1")(None)
    assert r1.extract_reasoning("still thinking") == ("still thinking", None)      # the start marker is implied
    r, c = _stream_reasoning(ReasoningParserManager.get_reasoning_parser("deepseek_r1")(None), "still thinking")
    assert (r, c) == ("still thinking", "")


def test_implicit_start_tolerates_an_explicit_one():
    text = "<think>thinking</think>answer"
    make = ReasoningParserManager.get_reasoning_parser("deepseek_r1")
    assert make(None).extract_reasoning(text) == ("thinking", "answer")
    assert _stream_reasoning(make(None), text) == ("thinking", "answer")


def test_delegating_parser_offline_and_streaming_agree():
    text = ('<think>need a tool</think>\n\nCalling. <tool_call>\n{"name": "f", "arguments": {"a": 1}}\n</tool_call>')
    make = lambda: DelegatingParser(ReasoningParserManager.get_reasoning_parser("qwen3")(None),      # noqa: E731
                                    ToolParserManager.get_tool_parser("hermes")(None))
    off = make().parse(text)
    assert off["reasoning_content"] == "need a tool" and off["content"] == "Calling."
    assert off["tool_calls"][0]["function"]["name"] == "f"
    d, r, c, calls = make(), "", "", []
    for i in range(1, len(text) + 1):
        o = d.parse_streaming(text[:i], final=i == len(text))
        r, c, calls = r + o["reasoning_content"], c + o["content"], calls + o["tool_calls"]
    assert r == "need a tool" and c.strip() == "Calling." and len(calls) == 1
    assert json.loads(calls[0]["function"]["arguments"]) == {"a": 1}
    # either half may be absent
    only_tools = DelegatingParser(None, ToolParserManager.get_tool_parser("hermes")(None)).parse(text)
    assert only_tools["reasoning_content"] is None and only_tools["tool_calls"]
    only_reason = DelegatingParser(ReasoningParserManager.get_reasoning_parser("qwen3")(None), None).parse(text)
    assert only_reason["tool_calls"] == [] and "<tool_call>" in only_reason["content"]


def test_detect_reasoning_parser():
    class Tok:
        def __init__(self, vocab):
            self.vocab = vocab

        def get_vocab(self):
            return self.vocab

    assert detect_reasoning_parser("qwen3_moe") == "qwen3"
    assert detect_reasoning_parser("deepseek_v3") == "deepseek_r1"
    assert detect_reasoning_parser("llama", Tok({"[THINK]": 1})) == "mistral"
    assert detect_reasoning_parser("llama", Tok({"<think>": 1})) == "qwen3"
    assert detect_reasoning_parser("llama", Tok({})) is None
    assert detect_reasoning_parser(None, None) is None
