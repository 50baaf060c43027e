from __future__ import annotations

import ast
import json
import re
import typing as tp
import uuid
from dataclasses import dataclass, field


@dataclass
class ExtractedToolCalls:
    tools_called: bool
    tool_calls: list[dict] = field(default_factory=list)   # OpenAI dicts: {id, type, function: {name, arguments}}
    content: str | None = None


def _call(name: str, args: tp.Any) -> dict:
    if not isinstance(args, str):
        args = json.dumps(args if args is not None else {}, ensure_ascii=False)
    return {"id": f"call-{uuid.uuid4().hex[:24]}", "type": "function", "function": {"name": name, "arguments": args}}


def _json_objects(text: str) -> list[tp.Any]:
    """All top-level JSON values found in ``text`` (objects or lists), skipping anything in between."""
    dec = json.JSONDecoder()
    out, i = [], 0
    while i < len(text):
        if text[i] in "{[":
            try:
                v, end = dec.raw_decode(text, i)
                out.append(v)
                i = end
                continue
            except json.JSONDecodeError:
                pass
        i += 1
    return out


def _coerce(v: str) -> tp.Any:
    s = v.strip()
    try:
        return json.loads(s)
    except (json.JSONDecodeError, ValueError):
        return v.strip("\n")


class ToolParser:
    """Base class. ``extract_tool_calls`` handles a finished generation; ``extract_tool_calls_streaming`` is fed
    the accumulated text after every delta and returns ``(content_delta, new_tool_calls)``."""

    start_markers: tuple[str, ...] = ()

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer
        self._sent_content = 0
        self._sent_calls = 0

    def extract_tool_calls(self, text: str, request=None) -> ExtractedToolCalls:
        raise NotImplementedError

    def _first_marker(self, text: str) -> int:
        idx = [text.find(m) for m in self.start_markers if m and m in text]
        return min(idx) if idx else -1

    def _partial_marker(self, text: str) -> int:
        """Length of the longest suffix of ``text`` that is a proper prefix of a start marker."""
        best = 0
        for m in self.start_markers:
            for n in range(min(len(m) - 1, len(text)), 0, -1):
                if text.endswith(m[:n]):
                    best = max(best, n)
                    break
        return best

    def extract_tool_calls_streaming(self, current_text: str, final: bool = False) -> tuple[str, list[dict]]:
        cut = self._first_marker(current_text)
        if cut < 0:
            safe = len(current_text) - (0 if final else self._partial_marker(current_text))
            delta = current_text[self._sent_content:safe]
            self._sent_content = max(self._sent_content, safe)
            return delta, []
        delta = current_text[self._sent_content:cut] if cut > self._sent_content else ""
        self._sent_content = max(self._sent_content, cut)
        res = self.extract_tool_calls(current_text)
        calls = res.tool_calls if res.tools_called else []
        n_ready = len(calls) if final else max(0, len(calls) - 1)   # the last call may still be growing
        new = calls[self._sent_calls:n_ready]
        for i, c in enumerate(new, start=self._sent_calls):
            c["index"] = i
        self._sent_calls = max(self._sent_calls, n_ready)
        return delta, new


class JsonTaggedParser(ToolParser):
    """JSON payload(s) after ``start`` (up to ``end`` when given). Objects use ``name_key`` / ``args_keys``."""

    def __init__(self, tokenizer=None, *, start: tuple[str, ...] = (), end: str | None = None, name_key="name",
                 args_keys=("arguments", "parameters"), bare_json: bool = False, strip_name_prefix: str = ""):
        super().__init__(tokenizer)
        self.start_markers, self.end = tuple(start), end
        self.name_key, self.args_keys, self.bare_json = name_key, tuple(args_keys), bare_json
        self.strip = strip_name_prefix

    def _to_calls(self, values) -> list[dict]:
        calls = []
        for v in values:
            for obj in (v if isinstance(v, list) else [v]):
                if not isinstance(obj, dict):
                    continue
                fn = obj.get("function") if isinstance(obj.get("function"), dict) else obj
                name = fn.get(self.name_key)
                if not isinstance(name, str):
                    continue
                args = next((fn[k] for k in self.args_keys if k in fn), {})
                calls.append(_call(name[len(self.strip):] if self.strip and name.startswith(self.strip) else name, args))
        return calls

    def extract_tool_calls(self, text, request=None):
        cut = self._first_marker(text)
        if cut < 0:
            if not self.bare_json:
                return ExtractedToolCalls(False, [], text)
            stripped = text.lstrip()
            if not stripped.startswith(("{", "[")):
                return ExtractedToolCalls(False, [], text)
            calls = self._to_calls(_json_objects(stripped))
            return ExtractedToolCalls(bool(calls), calls, None if calls else text)
        body = text[cut:]
        if self.end:
            parts = []
            for m in self.start_markers:
                for seg in body.split(m)[1:]:
                    parts.append(seg.split(self.end)[0])
            body = "\n".join(parts) if parts else body
        calls = self._to_calls(_json_objects(body))
        content = text[:cut].strip() or None
        return ExtractedToolCalls(bool(calls), calls, content if calls else text)


class XmlParamParser(ToolParser):
    """``<function=NAME> <parameter=K>V</parameter> ...`` style blocks described by three regular expressions."""

    def __init__(self, tokenizer=None, *, start: tuple[str, ...], call_rx: str, param_rx: str):
        super().__init__(tokenizer)
        self.start_markers = tuple(start)
        self.call_rx, self.param_rx = re.compile(call_rx, re.S), re.compile(param_rx, re.S)

    def extract_tool_calls(self, text, request=None):
        cut = self._first_marker(text)
        if cut < 0:
            return ExtractedToolCalls(False, [], text)
        calls = []
        for m in self.call_rx.finditer(text[cut:]):
            name, body = m.group("name").strip(), m.group("body")
            args = {p.group("key").strip(): _coerce(p.group("value")) for p in self.param_rx.finditer(body)}
            calls.append(_call(name, args))
        return ExtractedToolCalls(bool(calls), calls, (text[:cut].strip() or None) if calls else text)


class PythonicParser(ToolParser):
    """``[get_weather(city="Paris"), add(a=1, b=2)]`` (optionally inside wrapper tags)."""

    def __init__(self, tokenizer=None, *, start: tuple[str, ...] = ("[",), wrapper: tuple[str, str] | None = None):
        super().__init__(tokenizer)
        self.start_markers, self.wrapper = tuple(start), wrapper

    def extract_tool_calls(self, text, request=None):
        src = text.strip()
        lead = None
        if self.wrapper:
            a, b = self.wrapper
            if a not in src:
                return ExtractedToolCalls(False, [], text)
            lead = src.split(a)[0].strip() or None
            src = src.split(a, 1)[1].split(b)[0].strip()
            if not src.startswith("["):
                src = "[" + ",".join(l for l in src.splitlines() if l.strip()) + "]"
        i = src.find("[")
        if i < 0:
            return ExtractedToolCalls(False, [], text)
        lead = lead or (src[:i].strip() or None)
        try:
            tree = ast.parse(src[i:].strip(), mode="eval").body
        except SyntaxError:
            return ExtractedToolCalls(False, [], text)
        if not isinstance(tree, ast.List) or not tree.elts or not all(isinstance(e, ast.Call) for e in tree.elts):
            return ExtractedToolCalls(False, [], text)
        calls = []
        for e in tree.elts:
            try:
                name = ast.unparse(e.func)
                args = {k.arg: ast.literal_eval(k.value) for k in e.keywords}
            except (ValueError, SyntaxError):
                return ExtractedToolCalls(False, [], text)
            calls.append(_call(name, args))
        return ExtractedToolCalls(True, calls, lead)


class KeyValueBlockParser(ToolParser):
    """GLM-4.5 style: ``<tool_call>NAME\\n<arg_key>k</arg_key>\\n<arg_value>v</arg_value>...</tool_call>``."""

    start_markers = ("<tool_call>",)
    _blk = re.compile(r"<tool_call>\s*([^\n<]+)\s*(.*?)</tool_call>", re.S)
    _kv = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)

    def extract_tool_calls(self, text, request=None):
        calls = [_call(m.group(1).strip(), {k.strip(): _coerce(v) for k, v in self._kv.findall(m.group(2))})
                 for m in self._blk.finditer(text)]
        cut = text.find("<tool_call>")
        return ExtractedToolCalls(bool(calls), calls, (text[:cut].strip() or None) if calls else text)


class DeepSeekV3Parser(ToolParser):
    start_markers = ("<｜tool▁calls▁begin｜>",)
    _v3 = re.compile(r"<｜tool▁call▁begin｜>(?P<type>.*?)<｜tool▁sep｜>(?P<name>.*?)\n```json\n(?P<args>.*?)\n```"
                     r"\s*<｜tool▁call▁end｜>", re.S)
    _v31 = re.compile(r"<｜tool▁call▁begin｜>(?P<name>.*?)<｜tool▁sep｜>(?P<args>.*?)<｜tool▁call▁end｜>", re.S)

    def __init__(self, tokenizer=None, v31: bool = False):
        super().__init__(tokenizer)
        self.rx = self._v31 if v31 else self._v3

    def extract_tool_calls(self, text, request=None):
        cut = self._first_marker(text)
        if cut < 0:
            return ExtractedToolCalls(False, [], text)
        calls = [_call(m.group("name").strip(), m.group("args").strip()) for m in self.rx.finditer(text[cut:])]
        return ExtractedToolCalls(bool(calls), calls, (text[:cut].strip() or None) if calls else text)


class KimiK2Parser(ToolParser):
    start_markers = ("<|tool_calls_section_begin|>", "<|tool_call_section_begin|>")
    _rx = re.compile(r"<\|tool_call_begin\|>\s*(?P<id>[\w\.\-]+:\d+)\s*<\|tool_call_argument_begin\|>\s*"
                     r"(?P<args>.*?)\s*<\|tool_call_end\|>", re.S)

    def extract_tool_calls(self, text, request=None):
        cut = self._first_marker(text)
        if cut < 0:
            return ExtractedToolCalls(False, [], text)
        calls = []
        for m in self._rx.finditer(text[cut:]):
            c = _call(m.group("id").split(":")[0].split(".")[-1], m.group("args"))
            c["id"] = m.group("id")
            calls.append(c)
        return ExtractedToolCalls(bool(calls), calls, (text[:cut].strip() or None) if calls else text)


class HarmonyParser(ToolParser):
    """gpt-oss: ``<|channel|>commentary to=functions.NAME <|constrain|>json<|message|>{...}<|call|>``."""

    start_markers = ("to=functions.",)
    _rx = re.compile(r"to=functions\.(?P<name>[\w\-\.]+).*?<\|message\|>(?P<args>.*?)(?:<\|call\|>|<\|end\|>|$)", re.S)
    _final = re.compile(r"<\|channel\|>final<\|message\|>(.*?)(?:<\|return\|>|<\|end\|>|$)", re.S)

    def extract_tool_calls(self, text, request=None):
        calls = [_call(m.group("name"), m.group("args").strip()) for m in self._rx.finditer(text)]
        fin = self._final.search(text)
        content = fin.group(1).strip() if fin else (None if calls else text)
        return ExtractedToolCalls(bool(calls), calls, content)

    _done = re.compile(r"to=functions\.(?P<name>[\w\-\.]+).*?<\|message\|>(?P<args>.*?)(?:<\|call\|>|<\|end\|>)", re.S)

    def extract_tool_calls_streaming(self, current_text, final=False):
        # Channel markup is never content: only the text of the final channel streams out, and a call is reported
        # once its closing marker has arrived (or the generation ended).
        text = current_text
        if not final:
            hold = 0
            for m in ("<|channel|>", "<|message|>", "<|return|>", "<|end|>", "<|call|>", "<|start|>", "<|constrain|>"):
                for n in range(min(len(m) - 1, len(text)), 0, -1):
                    if text.endswith(m[:n]):
                        hold = max(hold, n)
                        break
            text = text[:len(text) - hold] if hold else text
        fin = self._final.search(text)
        if fin:
            content = fin.group(1).lstrip()
        else:
            content = "" if "<|" in text else text
        delta = content[self._sent_content:]
        self._sent_content = max(self._sent_content, len(content))
        rx = self._rx if final else self._done
        calls = [_call(m.group("name"), m.group("args").strip()) for m in rx.finditer(text)]
        new = calls[self._sent_calls:]
        for i, c in enumerate(new, start=self._sent_calls):
            c["index"] = i
        self._sent_calls = max(self._sent_calls, len(calls))
        return delta, new


class FunctionGemmaParser(ToolParser):
    """``<start_function_call>call:NAME{key:<escape>text<escape>,n:3}<end_function_call>``."""

    def __init__(self, tokenizer=None, start="<start_function_call>", end="<end_function_call>"):
        super().__init__(tokenizer)
        self.start_markers = (start,)
        self._rx = re.compile(re.escape(start) + r"\s*call:(?P<name>[\w\-\.]+)\s*\{(?P<body>.*?)\}\s*" + re.escape(end),
                              re.S)
        self._kv = re.compile(r"(\w+)\s*:\s*(?:<escape>(.*?)<escape>|([^,]*))", re.S)

    def extract_tool_calls(self, text, request=None):
        calls = []
        for m in self._rx.finditer(text):
            args = {k: (s if s != "" or raw == "" else _coerce(raw)) if s else _coerce(raw)
                    for k, s, raw in self._kv.findall(m.group("body"))}
            calls.append(_call(m.group("name"), args))
        cut = self._first_marker(text)
        return ExtractedToolCalls(bool(calls), calls, (text[:cut].strip() or None) if calls else text)


_XML_FN = dict(call_rx=r"<function=(?P<name>[^>\n]+)>(?P<body>.*?)</function>",
               param_rx=r"<parameter=(?P<key>[^>\n]+)>\n?(?P<value>.*?)\n?</parameter>")
_INVOKE = dict(call_rx=r"<invoke name=\"(?P<name>[^\"]+)\">(?P<body>.*?)</invoke>",
               param_rx=r"<parameter name=\"(?P<key>[^\"]+)\">(?P<value>.*?)</parameter>")

_TABLE: dict[str, tp.Callable[[tp.Any], ToolParser]] = {
    "hermes": lambda t: JsonTaggedParser(t, start=("<tool_call>",), end="</tool_call>"),
    "qwen": lambda t: JsonTaggedParser(t, start=("<tool_call>",), end="</tool_call>"),
    "ernie45": lambda t: JsonTaggedParser(t, start=("<tool_call>",), end="</tool_call>"),
    "longcat": lambda t: JsonTaggedParser(t, start=("<longcat_tool_call>",), end="</longcat_tool_call>"),
    "llama3_json": lambda t: JsonTaggedParser(t, start=("<|python_tag|>",), bare_json=True),
    "llama4_json": lambda t: JsonTaggedParser(t, start=("<|python_tag|>",), bare_json=True),
    "mistral": lambda t: JsonTaggedParser(t, start=("[TOOL_CALLS]",)),
    "granite": lambda t: JsonTaggedParser(t, start=("<|tool_call|>", "<tool_call>")),
    "granite-20b-fc": lambda t: JsonTaggedParser(t, start=("<function_call>",)),
    "internlm": lambda t: JsonTaggedParser(t, start=("<|action_start|><|plugin|>",), end="<|action_end|>"),
    "jamba": lambda t: JsonTaggedParser(t, start=("<tool_calls>",), end="</tool_calls>"),
    "hunyuan_a13b": lambda t: JsonTaggedParser(t, start=("<tool_calls>",), end="</tool_calls>"),
    "minimax": lambda t: JsonTaggedParser(t, start=("<tool_calls>",), end="</tool_calls>"),
    "xlam": lambda t: JsonTaggedParser(t, start=("```json", "[TOOL_CALLS]", "<tool_call>"), bare_json=True),
    "phi4_mini_json": lambda t: JsonTaggedParser(t, start=("functools",)),
    "gigachat3": lambda t: JsonTaggedParser(t, start=("function call",)),
    "custom": lambda t: JsonTaggedParser(t, start=("<tool_call>",), end="</tool_call>", bare_json=True),
    "qwen3_xml": lambda t: XmlParamParser(t, start=("<tool_call>", "<function="), **_XML_FN),
    "qwen3_coder": lambda t: XmlParamParser(t, start=("<tool_call>", "<function="), **_XML_FN),
    "step3p5": lambda t: XmlParamParser(t, start=("<tool_call>", "<function="), **_XML_FN),
    "seed_oss": lambda t: XmlParamParser(t, start=("<seed:tool_call>",), **_XML_FN),
    "minimax_m2": lambda t: XmlParamParser(t, start=("<minimax:tool_call>",), **_INVOKE),
    "deepseek_v32": lambda t: XmlParamParser(
        t, start=("<｜DSML｜function_calls>",),
        call_rx=r"<｜DSML｜invoke name=\"(?P<name>[^\"]+)\">(?P<body>.*?)</｜DSML｜invoke>",
        param_rx=r"<｜DSML｜parameter name=\"(?P<key>[^\"]+)\"[^>]*>(?P<value>.*?)</｜DSML｜parameter>"),
    "step3": lambda t: XmlParamParser(
        t, start=("<｜tool_calls_begin｜>",),
        call_rx=r"<steptml:invoke name=\"(?P<name>[^\"]+)\">(?P<body>.*?)</steptml:invoke>",
        param_rx=r"<steptml:parameter name=\"(?P<key>[^\"]+)\">(?P<value>.*?)</steptml:parameter>"),
    "pythonic": lambda t: PythonicParser(t),
    "llama4_pythonic": lambda t: PythonicParser(t, start=("[", "<|python_start|>")),
    "olmo3": lambda t: PythonicParser(t, start=("<function_calls>",), wrapper=("<function_calls>", "</function_calls>")),
    "glm45": lambda t: KeyValueBlockParser(t),
    "glm-4.5": lambda t: KeyValueBlockParser(t),
    "glm47": lambda t: KeyValueBlockParser(t),
    "glm-4.7": lambda t: KeyValueBlockParser(t),
    "deepseek_v3": lambda t: DeepSeekV3Parser(t, v31=False),
    "deepseek_v31": lambda t: DeepSeekV3Parser(t, v31=True),
    "kimi_k2": lambda t: KimiK2Parser(t),
    "openai": lambda t: HarmonyParser(t),
    "functiongemma": lambda t: FunctionGemmaParser(t),
    "gemma4": lambda t: FunctionGemmaParser(t, start="<|tool_call>", end="<tool_call|>"),
}

_BY_MODEL_TYPE = {
    "qwen2": "hermes", "qwen3": "hermes", "qwen3_moe": "hermes", "qwen2_moe": "hermes", "qwen3_next": "qwen3_coder",
    "llama": "llama3_json", "llama4": "llama4_pythonic", "mistral": "mistral", "mixtral": "mistral",
    "deepseek_v3": "deepseek_v3", "deepseek_v2": "deepseek_v3", "glm4_moe": "glm45", "glm4": "glm45",
    "granite": "granite", "granitemoe": "granite", "internlm2": "internlm", "jamba": "jamba", "phi3": "phi4_mini_json",
    "gpt_oss": "openai", "kimi_k2": "kimi_k2", "minimax": "minimax", "minimax_m2": "minimax_m2", "olmo3": "olmo3",
    "seed_oss": "seed_oss", "hunyuan": "hunyuan_a13b", "gemma3": "pythonic", "gemma3_text": "pythonic",
    "xlam": "xlam", "ernie4_5": "ernie45",
}


class ToolParserManager:
    @staticmethod
    def names() -> list[str]:
        return sorted(_TABLE)

    @staticmethod
    def get_tool_parser(name: str) -> tp.Callable[[tp.Any], ToolParser]:
        if name not in _TABLE:
            raise KeyError(f"unknown tool parser {name!r}; known: {sorted(_TABLE)}")
        return _TABLE[name]

    @staticmethod
    def register(name: str | list[str], factory: tp.Callable[[tp.Any], ToolParser]) -> None:
        for n in ([name] if isinstance(name, str) else name):
            _TABLE[n] = factory


def detect_tool_parser(model_type: str | None = None, tokenizer=None) -> str | None:
    """Picks a parser from the model type, else from marker tokens present in the tokenizer's vocabulary."""
    if model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    vocab = {}
    try:
        vocab = tokenizer.get_vocab() if tokenizer is not None else {}
    except Exception:
        pass
    for marker, name in (("<｜tool▁calls▁begin｜>", "deepseek_v3"), ("<|tool_calls_section_begin|>", "kimi_k2"),
                         ("[TOOL_CALLS]", "mistral"), ("<|python_tag|>", "llama3_json"), ("<tool_call>", "hermes")):
        if marker in vocab:
            return name
    return None
