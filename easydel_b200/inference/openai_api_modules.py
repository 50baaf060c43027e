"""OpenAI-compatible request / response schemas (easydel/inference/openai_api_modules.py, typed_models.py,
stream_protocol.py): chat completions, completions, the Responses API and the model list."""

from __future__ import annotations

import time
import typing as tp
import uuid

from pydantic import BaseModel, ConfigDict, Field


def _id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex[:24]}"


class _Open(BaseModel):
    model_config = ConfigDict(extra="allow")


class FunctionDefinition(_Open):
    name: str
    description: str | None = None
    parameters: dict | None = None


class ToolDefinition(_Open):
    type: str = "function"
    function: FunctionDefinition


class FunctionCall(_Open):
    name: str | None = None
    arguments: str | None = None


class ToolCall(_Open):
    id: str = Field(default_factory=lambda: _id("call"))
    type: str = "function"
    function: FunctionCall
    index: int | None = None


class ChatMessage(_Open):
    role: str
    content: str | list[dict] | None = None
    name: str | None = None
    tool_calls: list[ToolCall] | None = None
    tool_call_id: str | None = None
    reasoning_content: str | None = None


class DeltaMessage(_Open):
    role: str | None = None
    content: str | None = None
    reasoning_content: str | None = None
    tool_calls: list[ToolCall] | None = None


class UsageInfo(_Open):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0
    tokens_per_second: float | None = None
    processing_time: float | None = None
    time_to_first_token: float | None = None
    cached_tokens: int | None = None


class _SamplingFields(_Open):
    model: str | None = None
    max_tokens: int | None = None
    max_completion_tokens: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    n: int = 1
    stop: str | list[str] | None = None
    stream: bool = False
    stream_options: dict | None = None
    presence_penalty: float | None = None
    frequency_penalty: float | None = None
    repetition_penalty: float | None = None
    seed: int | None = None
    logit_bias: dict[str, float] | None = None
    logprobs: bool | int | None = None
    top_logprobs: int | None = None
    user: str | None = None
    ignore_eos: bool | None = None
    min_tokens: int | None = None
    stop_token_ids: list[int] | None = None

    def to_sampling_params(self, default_max_tokens: int = 256):
        from .sampling_params import SamplingParams

        mt = self.max_completion_tokens or self.max_tokens or default_max_tokens
        kw = dict(max_tokens=mt, n=self.n, stop=self.stop, seed=self.seed)
        for k in ("temperature", "top_p", "top_k", "min_p", "presence_penalty", "frequency_penalty",
                  "repetition_penalty", "ignore_eos", "min_tokens", "stop_token_ids"):
            v = getattr(self, k)
            if v is not None:
                kw[k] = v
        if self.logit_bias:
            kw["logit_bias"] = {int(k): float(v) for k, v in self.logit_bias.items()}
        return SamplingParams(**kw)


class ChatCompletionRequest(_SamplingFields):
    messages: list[ChatMessage]
    tools: list[ToolDefinition] | None = None
    tool_choice: str | dict | None = None
    response_format: dict | None = None
    chat_template_kwargs: dict | None = None
    add_generation_prompt: bool = True


class ChatCompletionResponseChoice(_Open):
    index: int = 0
    message: ChatMessage
    finish_reason: str | None = None
    logprobs: dict | None = None


class ChatCompletionResponse(_Open):
    id: str = Field(default_factory=lambda: _id("chatcmpl"))
    object: str = "chat.completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: list[ChatCompletionResponseChoice] = []
    usage: UsageInfo = UsageInfo()


class ChatCompletionStreamResponseChoice(_Open):
    index: int = 0
    delta: DeltaMessage
    finish_reason: str | None = None


class ChatCompletionStreamResponse(_Open):
    id: str = Field(default_factory=lambda: _id("chatcmpl"))
    object: str = "chat.completion.chunk"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: list[ChatCompletionStreamResponseChoice] = []
    usage: UsageInfo | None = None


class CompletionRequest(_SamplingFields):
    prompt: str | list[str] | list[int] | list[list[int]]
    echo: bool = False
    suffix: str | None = None


class CompletionResponseChoice(_Open):
    index: int = 0
    text: str = ""
    finish_reason: str | None = None
    logprobs: dict | None = None


class CompletionResponse(_Open):
    id: str = Field(default_factory=lambda: _id("cmpl"))
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: list[CompletionResponseChoice] = []
    usage: UsageInfo = UsageInfo()


class CompletionStreamResponse(CompletionResponse):
    object: str = "text_completion"
    usage: UsageInfo | None = None


class ResponsesRequest(_SamplingFields):
    input: str | list[dict]
    instructions: str | None = None
    previous_response_id: str | None = None
    store: bool = True
    tools: list[dict] | None = None
    max_output_tokens: int | None = None
    reasoning: dict | None = None


class ResponsesOutputText(_Open):
    type: str = "output_text"
    text: str = ""
    annotations: list = []


class ResponsesOutputItem(_Open):
    id: str = Field(default_factory=lambda: _id("msg"))
    type: str = "message"
    role: str = "assistant"
    status: str = "completed"
    content: list[ResponsesOutputText] = []


class ResponsesResponse(_Open):
    id: str = Field(default_factory=lambda: _id("resp"))
    object: str = "response"
    created_at: int = Field(default_factory=lambda: int(time.time()))
    status: str = "completed"
    model: str = ""
    output: list[dict] = []
    output_text: str = ""
    previous_response_id: str | None = None
    usage: dict = {}


class ModelCard(_Open):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "easydel"
    max_model_len: int | None = None


class ModelList(_Open):
    object: str = "list"
    data: list[ModelCard] = []


class ToolExecuteRequest(_Open):
    name: str
    arguments: dict = {}


def sse(payload: BaseModel | dict | str) -> str:
    """One server-sent-events frame."""
    import json

    if isinstance(payload, BaseModel):
        data = payload.model_dump_json(exclude_none=True)
    elif isinstance(payload, str):
        data = payload
    else:
        data = json.dumps(payload)
    return f"data: {data}\n\n"
