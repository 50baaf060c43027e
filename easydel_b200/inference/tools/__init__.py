"""Tool-call parsers: turn model text into OpenAI ``tool_calls`` (easydel/inference/tools/parsers/*).

The reference ships one module per model family (33 of them). The formats fall into four mechanical groups:
JSON payloads between marker tokens, XML-ish ``function`` / ``parameter`` blocks, python call lists, and a few
one-off layouts, so the parsers here are instances of four small engines configured by a table. Names match the
reference's registry (``ToolParserManager.get_tool_parser("hermes")`` ...).
"""

from .parsers import (ExtractedToolCalls, ToolParser, ToolParserManager, detect_tool_parser)  # noqa: F401
