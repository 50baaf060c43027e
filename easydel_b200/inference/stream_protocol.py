"""Server-sent-event protocol of the Responses API, and the text-delta helper shared by the streaming endpoints
(easydel/inference/stream_protocol.py:123-162 for the delta rule, :556-1065 for the Responses event stream).

A streamed response is a sequence of typed events, each with a running ``sequence_number``:

    response.created, response.in_progress
    per output item, in the order the model produced them
        reasoning      output_item.added, reasoning_summary_part.added, reasoning_summary_text.delta*, .done,
                       reasoning_summary_part.done, output_item.done
        function_call  output_item.added, function_call_arguments.delta, .done, output_item.done
        message        output_item.added, content_part.added, output_text.delta*, output_text.done,
                       content_part.done, output_item.done
    response.completed                       (carries the whole response object, usage included)

:class:`ResponsesStreamBuilder` turns the parser's per-step deltas (reasoning text, visible text, finished tool calls)
into those events. An item is opened by its first delta and closed when another kind of output begins or the
generation ends, so reasoning -> tool call -> message comes out as three items with consecutive ``output_index``.
"""

from __future__ import annotations

import json
import time
import typing as tp
import uuid


def stream_delta(current_text: str, previous_text: str, fallback_delta: str = "") -> str:
    """What to send after ``previous_text`` was sent and the accumulated text now reads ``current_text``.

    The tail when one extends the other; otherwise (a parser rewrote a boundary) the part of ``current_text`` after
    the longest overlap between the end of what was sent and its beginning; ``fallback_delta`` (the engine's raw
    delta) when no overlap exists and it was not already sent; else nothing."""
    cur, prev, fb = current_text or "", previous_text or "", fallback_delta or ""
    if cur.startswith(prev):
        return cur[len(prev):]
    for n in range(min(len(prev), len(cur)), 0, -1):
        if prev.endswith(cur[:n]):
            return cur[n:]
    if fb and not prev.endswith(fb):
        return fb
    return ""


def sse_frame(event: str | None, payload: tp.Any) -> str:
    """One server-sent event: an optional ``event:`` line and a ``data:`` line holding JSON (or a literal string)."""
    data = payload if isinstance(payload, str) else json.dumps(payload, ensure_ascii=False, separators=(",", ":"))
    head = f"event: {event}\n" if event else ""
    return f"{head}data: {data}\n\n"


def _new_id(prefix: str) -> str:
    return f"{prefix}_{uuid.uuid4().hex[:24]}"


class ResponsesStreamBuilder:
    """Single-use: ``start()``, ``feed()`` once per engine step, ``finish()``. Every call returns the list of
    ``(event_name, payload)`` pairs to send; ``finish`` also returns the final response object."""

    def __init__(self, response_id: str | None = None, model: str = "", previous_response_id: str | None = None,
                 created_at: int | None = None):
        self.response_id = response_id or _new_id("resp")
        self.model, self.previous_response_id = model, previous_response_id
        self.created_at = int(created_at if created_at is not None else time.time())
        self.items: list[dict] = []          # finished output items, in order
        self._seq = 0
        self._open: dict | None = None       # the item that is receiving deltas
        self._finished = False

    # ------------------------------------------------------------------ plumbing
    def _event(self, name: str, **payload) -> tuple[str, dict]:
        ev = {"type": name, "sequence_number": self._seq, **payload}
        self._seq += 1
        return name, ev

    def _skeleton(self, status: str, usage: dict | None = None) -> dict:
        text = "".join(p["text"] for it in self.items if it["type"] == "message" for p in it["content"])
        return {"id": self.response_id, "object": "response", "created_at": self.created_at, "status": status,
                "model": self.model, "output": list(self.items), "output_text": text,
                "previous_response_id": self.previous_response_id, "usage": usage}

    def _close(self) -> list[tuple[str, dict]]:
        it, out = self._open, []
        if it is None:
            return out
        idx, kind = it["index"], it["item"]["type"]
        if kind == "reasoning":
            part = {"type": "summary_text", "text": it["text"]}
            it["item"]["summary"] = [part]
            out.append(self._event("response.reasoning_summary_text.done", item_id=it["item"]["id"],
                                   output_index=idx, summary_index=0, text=it["text"]))
            out.append(self._event("response.reasoning_summary_part.done", item_id=it["item"]["id"],
                                   output_index=idx, summary_index=0, part=part))
        elif kind == "message":
            part = {"type": "output_text", "text": it["text"], "annotations": []}
            it["item"]["content"] = [part]
            out.append(self._event("response.output_text.done", item_id=it["item"]["id"], output_index=idx,
                                   content_index=0, text=it["text"]))
            out.append(self._event("response.content_part.done", item_id=it["item"]["id"], output_index=idx,
                                   content_index=0, part=part))
        it["item"]["status"] = "completed"
        out.append(self._event("response.output_item.done", output_index=idx, item=dict(it["item"])))
        self.items.append(it["item"])
        self._open = None
        return out

    def _open_item(self, kind: str) -> list[tuple[str, dict]]:
        out = self._close()
        idx = len(self.items)
        if kind == "reasoning":
            item = {"id": _new_id("rs"), "type": "reasoning", "status": "in_progress", "summary": []}
        else:
            item = {"id": _new_id("msg"), "type": "message", "role": "assistant", "status": "in_progress",
                    "content": []}
        self._open = {"index": idx, "item": item, "text": ""}
        out.append(self._event("response.output_item.added", output_index=idx, item=dict(item)))
        if kind == "reasoning":
            out.append(self._event("response.reasoning_summary_part.added", item_id=item["id"], output_index=idx,
                                   summary_index=0, part={"type": "summary_text", "text": ""}))
        else:
            out.append(self._event("response.content_part.added", item_id=item["id"], output_index=idx,
                                   content_index=0, part={"type": "output_text", "text": "", "annotations": []}))
        return out

    # ------------------------------------------------------------------ life cycle
    def start(self) -> list[tuple[str, dict]]:
        return [self._event("response.created", response=self._skeleton("in_progress")),
                self._event("response.in_progress", response=self._skeleton("in_progress"))]

    def feed(self, reasoning_delta: str = "", content_delta: str = "",
             tool_calls: tp.Sequence[dict] = ()) -> list[tuple[str, dict]]:
        if self._finished:
            raise RuntimeError("the stream was already finished")
        out: list[tuple[str, dict]] = []
        if reasoning_delta:
            if self._open is None or self._open["item"]["type"] != "reasoning":
                out += self._open_item("reasoning")
            self._open["text"] += reasoning_delta
            out.append(self._event("response.reasoning_summary_text.delta", item_id=self._open["item"]["id"],
                                   output_index=self._open["index"], summary_index=0, delta=reasoning_delta))
        for call in tool_calls:
            out += self._close()
            fn = call.get("function", call)
            args = fn.get("arguments", "")
            if not isinstance(args, str):
                args = json.dumps(args, ensure_ascii=False, separators=(",", ":"))
            idx = len(self.items)
            item = {"id": _new_id("fc"), "type": "function_call", "status": "in_progress",
                    "call_id": call.get("id") or _new_id("call"), "name": fn.get("name", ""), "arguments": ""}
            out.append(self._event("response.output_item.added", output_index=idx, item=dict(item)))
            out.append(self._event("response.function_call_arguments.delta", item_id=item["id"], output_index=idx,
                                   delta=args))
            out.append(self._event("response.function_call_arguments.done", item_id=item["id"], output_index=idx,
                                   arguments=args))
            item.update(arguments=args, status="completed")
            out.append(self._event("response.output_item.done", output_index=idx, item=dict(item)))
            self.items.append(item)
        if content_delta:
            if self._open is None or self._open["item"]["type"] != "message":
                if not content_delta.strip() and self._open is None and self.items:
                    return out           # white space between two tool calls is not a message of its own
                out += self._open_item("message")
            self._open["text"] += content_delta
            out.append(self._event("response.output_text.delta", item_id=self._open["item"]["id"],
                                   output_index=self._open["index"], content_index=0, delta=content_delta))
        return out

    def finish(self, usage: dict | None = None, status: str = "completed") -> tuple[list[tuple[str, dict]], dict]:
        if self._finished:
            raise RuntimeError("the stream was already finished")
        out = self._close()
        if not any(it["type"] in ("message", "function_call") for it in self.items):
            out += self._open_item("message")           # a response always carries an assistant message
            out += self._close()
        self._finished = True
        final = self._skeleton(status, usage)
        out.append(self._event("response.completed" if status == "completed" else f"response.{status}",
                               response=final))
        return out, final


__all__ = ["stream_delta", "sse_frame", "ResponsesStreamBuilder"]
