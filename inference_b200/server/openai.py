"""OpenAI chat-completions wire format <-> the TextLlm contract (role of mlx-llm-server's openai.rs; its
behaviour: POST /v1/chat/completions with `messages`, `max_tokens`, `temperature`, `top_p`, `seed`, `stop`, `stream`,
`response_format: {"type": "json_object"}`, `tools`; responses `chat.completion` / `chat.completion.chunk`)."""
from __future__ import annotations

import json
import time
import uuid
from typing import Any

from ..contracts.core_llm import Constraint, Message, Role, Sampling, TextLlmOutput, TextLlmRequest
from ..contracts.core_llm.output import Channel, DoneEvent, FinishReason, TokenEvent
from ..contracts.errors import InvalidRequest

DEFAULT_MAX_TOKENS = 512
_ROLES = {"system": Role.SYSTEM, "user": Role.USER, "assistant": Role.ASSISTANT, "tool": Role.TOOL}


def _content_text(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if isinstance(content, list):      # [{"type": "text", "text": ...}, ...]
        parts = []
        for p in content:
            if not isinstance(p, dict) or p.get("type") != "text":
                raise InvalidRequest("only text content parts are supported")
            parts.append(str(p.get("text", "")))
        return "".join(parts)
    raise InvalidRequest("message content must be a string or a list of content parts")


def _number(j: dict, key: str, default, kind=float, lo=None):
    """A numeric request field: absent -> default; null, a string, a list, a bool or a non-finite value -> 400."""
    if key not in j:
        return default
    v = j[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != v or v in (float("inf"), float("-inf")):
        raise InvalidRequest(f"`{key}` must be a number")
    if kind is int and int(v) != v:
        raise InvalidRequest(f"`{key}` must be an integer")
    if lo is not None and v < lo:
        raise InvalidRequest(f"`{key}` must be >= {lo}")
    return kind(v)


def parse_chat_request(body: bytes) -> tuple[TextLlmRequest, bool, str | None]:
    """-> (request, stream, requested model id). Raises InvalidRequest on malformed input."""
    try:
        j = json.loads(body.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise InvalidRequest(f"request body is not valid JSON: {e}")
    if not isinstance(j, dict) or not isinstance(j.get("messages"), list) or not j["messages"]:
        raise InvalidRequest("`messages` must be a non-empty list")
    msgs = []
    for m in j["messages"]:
        role = _ROLES.get(m.get("role") if isinstance(m, dict) else None)
        if role is None:
            raise InvalidRequest(f"unknown message role {m.get('role') if isinstance(m, dict) else m!r}")
        msgs.append(Message.text(role, _content_text(m.get("content"))))
    temp = _number(j, "temperature", 1.0)
    top_p = _number(j, "top_p", 1.0, lo=0.0)
    top_k = _number(j, "top_k", 0, int, lo=0)
    rep = _number(j, "repetition_penalty", 1.0, lo=0.0)
    sampling = Sampling.greedy() if temp <= 0 else Sampling(temperature=temp, top_p=top_p, top_k=top_k,
                                                            repetition_penalty=rep)
    if j.get("seed") is not None and (isinstance(j["seed"], bool) or not isinstance(j["seed"], int)):
        raise InvalidRequest("`seed` must be an integer")
    if not isinstance(j.get("stop") or [], (str, list)):
        raise InvalidRequest("`stop` must be a string or a list of strings")
    stop = j.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    max_tokens = j.get("max_completion_tokens", j.get("max_tokens", DEFAULT_MAX_TOKENS))
    if not isinstance(max_tokens, int) or max_tokens < 1:
        raise InvalidRequest("`max_tokens` must be a positive integer")
    rf = j.get("response_format") or {}
    constraint = Constraint.JSON if isinstance(rf, dict) and rf.get("type") == "json_object" else None
    tools = []
    if j.get("tools"):
        from ..contracts.core_llm import ToolSpec

        for t in j["tools"]:
            f = t.get("function", {}) if isinstance(t, dict) else {}
            if not f.get("name"):
                raise InvalidRequest("every tool needs function.name")
            tools.append(ToolSpec(f["name"], f.get("description", ""), f.get("parameters") or {}))
    req = TextLlmRequest(messages=msgs, max_new_tokens=max_tokens, sampling=sampling, seed=j.get("seed"),
                         constraint=constraint, tools=tools, stop=[str(s) for s in stop])
    return req, bool(j.get("stream", False)), j.get("model")


def _finish(reason: FinishReason | None, has_tools: bool) -> str:
    if has_tools:
        return "tool_calls"
    return {FinishReason.STOP: "stop", FinishReason.LENGTH: "length", FinishReason.CANCELLED: "stop",
            FinishReason.CONTENT_FILTER: "content_filter", None: "stop"}[reason]


def completion_id() -> str:
    return "chatcmpl-" + uuid.uuid4().hex[:24]


def completion_body(cid: str, model: str, out: TextLlmOutput) -> dict:
    msg: dict[str, Any] = {"role": "assistant", "content": out.text}
    if out.thinking:
        msg["reasoning_content"] = out.thinking
    if out.tool_calls:
        msg["tool_calls"] = [{"id": f"call_{i}", "type": "function",
                              "function": {"name": c.name, "arguments": json.dumps(c.arguments)}}
                             for i, c in enumerate(out.tool_calls)]
    return {"id": cid, "object": "chat.completion", "created": int(time.time()), "model": model,
            "choices": [{"index": 0, "message": msg, "finish_reason": _finish(out.finish_reason, bool(out.tool_calls))}],
            "usage": {"prompt_tokens": out.usage.prompt_tokens, "completion_tokens": out.usage.generated_tokens,
                      "total_tokens": out.usage.total_tokens()}}


def chunk_body(cid: str, model: str, event, first: bool) -> dict | None:
    base = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model}
    if isinstance(event, TokenEvent):
        delta: dict[str, Any] = {"role": "assistant"} if first else {}
        delta["reasoning_content" if event.channel is Channel.THINKING else "content"] = event.text
        return {**base, "choices": [{"index": 0, "delta": delta, "finish_reason": None}]}
    if isinstance(event, DoneEvent):
        return {**base, "choices": [{"index": 0, "delta": {}, "finish_reason": _finish(event.finish_reason, False)}],
                "usage": {"prompt_tokens": event.usage.prompt_tokens, "completion_tokens": event.usage.generated_tokens,
                          "total_tokens": event.usage.total_tokens()}}
    return None


def error_body(message: str, kind: str = "invalid_request_error", code: str | None = None) -> dict:
    return {"error": {"message": message, "type": kind, "code": code}}
