"""Reasoning parsers: split model text into ``reasoning_content`` and ``content``
(easydel/inference/reasoning/parsers/*, 15 parsers in the reference).

Almost every family wraps its chain of thought in a start / end marker pair; the differences are the marker
strings and whether the start marker is implied by the chat template (DeepSeek-R1, Qwen3 thinking models emit
only the end marker). Parsers are therefore instances of :class:`DelimitedReasoningParser` configured by a table,
plus one parser for the channel layout of gpt-oss.
"""

from __future__ import annotations

import re
import typing as tp


class ReasoningParser:
    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer
        self._sent_r = self._sent_c = 0

    def extract_reasoning(self, text: str) -> tuple[str | None, str | None]:
        """``(reasoning, content)`` of a finished generation."""
        raise NotImplementedError

    def extract_reasoning_streaming(self, current_text: str, final: bool = False) -> tuple[str, str]:
        """Fed the accumulated text; returns the not-yet-sent ``(reasoning_delta, content_delta)``."""
        r, c = self._split_partial(current_text, final)
        dr, dc = r[self._sent_r:], c[self._sent_c:]
        self._sent_r, self._sent_c = max(self._sent_r, len(r)), max(self._sent_c, len(c))
        return dr, dc

    def _split_partial(self, text: str, final: bool) -> tuple[str, str]:
        r, c = self.extract_reasoning(text)
        return r or "", c or ""


def _hold_back(text: str, markers: tp.Sequence[str]) -> int:
    """Number of trailing characters that could be the beginning of a marker (not safe to stream yet)."""
    best = 0
    for m in markers:
        for n in range(min(len(m) - 1, len(text)), 0, -1):
            if text.endswith(m[:n]):
                best = max(best, n)
                break
    return best


class DelimitedReasoningParser(ReasoningParser):
    def __init__(self, tokenizer=None, *, start: str, end: str, implicit_start: bool = False,
                 content_start: str | None = None, content_end: str | None = None):
        super().__init__(tokenizer)
        self.start, self.end, self.implicit = start, end, implicit_start
        self.cs, self.ce = content_start, content_end

    def _clean_content(self, c: str) -> str:
        if self.cs and self.cs in c:
            c = c.split(self.cs, 1)[1]
        if self.ce and self.ce in c:
            c = c.split(self.ce, 1)[0]
        return c

    def extract_reasoning(self, text):
        if self.start in text:
            pre, rest = text.split(self.start, 1)
            if self.end in rest:
                r, c = rest.split(self.end, 1)
                return r.strip("\n") or None, (self._clean_content(pre + c).lstrip("\n") or None)
            return rest.strip("\n") or None, (pre or None)
        if self.implicit and self.end in text:
            r, c = text.split(self.end, 1)
            return r.strip("\n") or None, (self._clean_content(c).lstrip("\n") or None)
        if self.implicit:
            return text or None, None
        return None, self._clean_content(text) or None

    def _split_partial(self, text, final):
        # Markers are located in the whole text first; only the open stream's tail is held back while it could be
        # the beginning of a marker. Trimming the text before the search would cut a complete marker whose last
        # characters begin another one ("\n</think>\n" ends in the first character of "\n</answer>").
        def trim(s, markers):
            n = 0 if final else _hold_back(s, markers)
            return s[:len(s) - n] if n else s

        cm = [m for m in (self.cs, self.ce) if m]
        if self.start in text:
            pre, body = text.split(self.start, 1)
            in_reasoning = True
        else:
            pre, body, in_reasoning = "", text, self.implicit
        if not in_reasoning:
            return "", trim(self._clean_content(body), [self.start] + cm)
        if self.end in body:
            r, c = body.split(self.end, 1)
            return r, trim(self._clean_content(pre + c).lstrip("\n"), cm)
        return trim(body, [self.end] if pre or self.start in text else [self.end, self.start]), pre


class HarmonyReasoningParser(ReasoningParser):
    """gpt-oss: ``<|channel|>analysis<|message|>...<|end|>`` is reasoning, the ``final`` channel is content."""

    _ana = re.compile(r"<\|channel\|>analysis<\|message\|>(.*?)(?:<\|end\|>|<\|start\|>|$)", re.S)
    _fin = re.compile(r"<\|channel\|>final<\|message\|>(.*?)(?:<\|return\|>|<\|end\|>|$)", re.S)

    def extract_reasoning(self, text):
        a = "\n".join(m.strip() for m in self._ana.findall(text)) or None
        f = self._fin.search(text)
        if f:
            return a, f.group(1).strip() or None
        if a is None and "<|channel|>" not in text:
            return None, text or None
        return a, None

    _MARKS = ("<|channel|>", "<|message|>", "<|end|>", "<|start|>", "<|return|>", "<|call|>")

    def _split_partial(self, text, final):
        # no trailing strip while streaming: what was sent must stay a prefix of what is sent next
        if not final:
            n = _hold_back(text, self._MARKS)
            text = text[:len(text) - n] if n else text
        a = "\n".join(m.lstrip() for m in self._ana.findall(text))
        f = self._fin.search(text)
        if f:
            return a, f.group(1).lstrip()
        if not a and not any(m in text for m in self._MARKS):
            return "", text
        return a, ""


class IdentityReasoningParser(ReasoningParser):
    def extract_reasoning(self, text):
        return None, text or None


_THINK = dict(start="<think>", end="</think>")
_TABLE: dict[str, tp.Callable[[tp.Any], ReasoningParser]] = {
    "deepseek_r1": lambda t: DelimitedReasoningParser(t, **_THINK, implicit_start=True),
    "deepseek_v3": lambda t: DelimitedReasoningParser(t, **_THINK),
    "qwen3": lambda t: DelimitedReasoningParser(t, **_THINK),
    "qwen3_thinking": lambda t: DelimitedReasoningParser(t, **_THINK, implicit_start=True),
    "glm45": lambda t: DelimitedReasoningParser(t, **_THINK),
    "ernie45": lambda t: DelimitedReasoningParser(t, **_THINK, implicit_start=True,
                                                  content_start="<response>", content_end="</response>"),
    "minimax_m2": lambda t: DelimitedReasoningParser(t, **_THINK, implicit_start=True),
    "olmo3": lambda t: DelimitedReasoningParser(t, **_THINK, implicit_start=True),
    "step3": lambda t: DelimitedReasoningParser(t, **_THINK, implicit_start=True),
    "step3p5": lambda t: DelimitedReasoningParser(t, **_THINK, implicit_start=True),
    "mistral": lambda t: DelimitedReasoningParser(t, start="[THINK]", end="[/THINK]"),
    "seed_oss": lambda t: DelimitedReasoningParser(t, start="<seed:think>", end="</seed:think>"),
    "hunyuan_a13b": lambda t: DelimitedReasoningParser(t, start="<think>\n", end="\n</think>\n",
                                                       content_start="<answer>\n", content_end="\n</answer>"),
    "granite": lambda t: DelimitedReasoningParser(t, start="Here is my thought process:",
                                                  end="Here is my response:"),
    "gemma4": lambda t: DelimitedReasoningParser(t, start="<|channel>thought\n", end="<channel|>"),
    "gpt_oss": lambda t: HarmonyReasoningParser(t),
    "openai": lambda t: HarmonyReasoningParser(t),
    "identity": lambda t: IdentityReasoningParser(t),
}
_BY_MODEL_TYPE = {"qwen3": "qwen3", "qwen3_moe": "qwen3", "deepseek_v3": "deepseek_r1", "gpt_oss": "gpt_oss",
                  "glm4_moe": "glm45", "mistral": "mistral", "seed_oss": "seed_oss", "granite": "granite",
                  "olmo3": "olmo3", "minimax_m2": "minimax_m2", "ernie4_5": "ernie45", "hunyuan": "hunyuan_a13b"}


class ReasoningParserManager:
    @staticmethod
    def names() -> list[str]:
        return sorted(_TABLE)

    @staticmethod
    def get_reasoning_parser(name: str) -> tp.Callable[[tp.Any], ReasoningParser]:
        if name not in _TABLE:
            raise KeyError(f"unknown reasoning parser {name!r}; known: {sorted(_TABLE)}")
        return _TABLE[name]

    @staticmethod
    def register(name: str, factory) -> None:
        _TABLE[name] = factory


def detect_reasoning_parser(model_type: str | None = None, tokenizer=None) -> str | None:
    if model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    try:
        vocab = tokenizer.get_vocab() if tokenizer is not None else {}
    except Exception:
        vocab = {}
    for marker, name in (("<seed:think>", "seed_oss"), ("[THINK]", "mistral"), ("<think>", "qwen3")):
        if marker in vocab:
            return name
    return None


class DelegatingParser:
    """Runs the reasoning parser first and the tool parser on what remains (the reference's ``DelegatingParser``)."""

    def __init__(self, reasoning_parser: ReasoningParser | None = None, tool_parser=None):
        self.reasoning, self.tools = reasoning_parser, tool_parser
        self._content = ""

    def parse(self, text: str) -> dict:
        r, c = self.reasoning.extract_reasoning(text) if self.reasoning else (None, text)
        calls = []
        if self.tools is not None and c:
            ex = self.tools.extract_tool_calls(c)
            if ex.tools_called:
                c, calls = ex.content, ex.tool_calls
        return {"reasoning_content": r, "content": c, "tool_calls": calls}

    def parse_streaming(self, current_text: str, final: bool = False) -> dict:
        if self.reasoning:
            dr, dc = self.reasoning.extract_reasoning_streaming(current_text, final)
        else:
            dr, dc = "", current_text[len(self._content):]
        self._content += dc
        calls = []
        if self.tools is not None:
            dc, calls = self.tools.extract_tool_calls_streaming(self._content, final)
        return {"reasoning_content": dr, "content": dc, "tool_calls": calls}
