"""Tool (function) calling: specs, parsed calls and the streaming `<tool_call>` segmenter
(core-llm/src/tool.rs:32-253). Two body dialects are parsed: Hermes JSON `{"name":..,"arguments":{..}}`
and Qwen XML `<function=name><parameter=key>value</parameter></function>`; XML string values are coerced
to the schema's declared non-string types."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any

from .thinking import max_partial_suffix

OPEN = "<tool_call>"
CLOSE = "</tool_call>"


@dataclass
class ToolSpec:
    name: str
    description: str
    parameters: dict[str, Any]

    def to_template_json(self) -> dict[str, Any]:
        return {"type": "function",
                "function": {"name": self.name, "description": self.description, "parameters": self.parameters}}

    def param_types(self) -> dict[str, str]:
        props = self.parameters.get("properties") if isinstance(self.parameters, dict) else None
        out = {}
        if isinstance(props, dict):
            for k, schema in props.items():
                if isinstance(schema, dict) and isinstance(schema.get("type"), str):
                    out[k] = schema["type"]
        return out


@dataclass
class ToolCall:
    name: str = ""
    arguments: dict[str, Any] = field(default_factory=dict)

    def to_template_json(self) -> dict[str, Any]:
        return {"type": "function", "function": {"name": self.name, "arguments": self.arguments}}


def _parse_xml_call(body: str) -> ToolCall | None:
    FN, PARAM, PARAM_END = "<function=", "<parameter=", "</parameter>"
    i = body.find(FN)
    if i < 0:
        return None
    fstart = i + len(FN)
    nend = body.find(">", fstart)
    if nend < 0:
        return None
    name = body[fstart:nend].strip()
    if not name:
        return None
    args: dict[str, Any] = {}
    rest = body[nend + 1:]
    while True:
        ps = rest.find(PARAM)
        if ps < 0:
            break
        kstart = ps + len(PARAM)
        kend = rest.find(">", kstart)
        if kend < 0:
            return None
        key = rest[kstart:kend].strip()
        vend = rest.find(PARAM_END, kend + 1)
        if vend < 0:
            return None
        args[key] = rest[kend + 1:vend].strip()
        rest = rest[vend + len(PARAM_END):]
    return ToolCall(name, args)


def _parse_json_call(body: str) -> ToolCall | None:
    try:
        v = json.loads(body)
    except json.JSONDecodeError:
        return None
    if not isinstance(v, dict) or not isinstance(v.get("name"), str):
        return None
    a = v.get("arguments")
    if isinstance(a, dict):
        args = a
    elif isinstance(a, str):
        try:
            parsed = json.loads(a)
            args = parsed if isinstance(parsed, dict) else {}
        except json.JSONDecodeError:
            args = {}
    else:
        args = {}
    return ToolCall(v["name"], args)


class ToolCallSegmenter:
    """Splits streamed text into visible content and parsed tool calls; holds back partial markers."""

    def __init__(self, tools: list[ToolSpec]):
        self.schemas = {t.name: t.param_types() for t in tools}
        self._in_call = False
        self.pending = ""
        self.body = ""
        self._calls: list[ToolCall] = []

    def in_call(self) -> bool:
        return self._in_call

    def push(self, delta: str) -> list[str]:
        if self._in_call:
            self.body += delta
        else:
            self.pending += delta
        out: list[str] = []
        while True:
            if self._in_call:
                pos = self.body.find(CLOSE)
                if pos < 0:
                    break
                block, rest = self.body[:pos], self.body[pos + len(CLOSE):]
                self.body = ""
                call = self._parse_block(block)
                if call is not None:
                    self._calls.append(call)
                self.pending += rest
                self._in_call = False
                continue
            pos = self.pending.find(OPEN)
            if pos >= 0:
                if pos > 0:
                    out.append(self.pending[:pos])
                self.body += self.pending[pos + len(OPEN):]
                self.pending = ""
                self._in_call = True
                continue
            hold = max_partial_suffix(self.pending, OPEN)
            safe = len(self.pending) - hold
            if safe > 0:
                out.append(self.pending[:safe])
                self.pending = self.pending[safe:]
            break
        return out

    def flush(self) -> list[str]:
        out = []
        if self._in_call:
            body, self.body = self.body, ""
            call = self._parse_block(body)
            if call is not None:
                self._calls.append(call)
            elif body:
                out.append(OPEN + body)
            self._in_call = False
        if self.pending:
            out.append(self.pending)
            self.pending = ""
        return out

    def calls(self) -> list[ToolCall]:
        return self._calls

    def take_calls(self) -> list[ToolCall]:
        c, self._calls = self._calls, []
        return c

    def _parse_block(self, block: str) -> ToolCall | None:
        t = block.strip()
        if not t:
            return None
        call = _parse_json_call(t) if t.startswith("{") else _parse_xml_call(t)
        if call is None:
            return None
        types = self.schemas.get(call.name)
        if types is None:
            return call
        for k, v in list(call.arguments.items()):
            if isinstance(v, str) and types.get(k, "string") != "string":
                try:
                    call.arguments[k] = json.loads(v.strip())
                except json.JSONDecodeError:
                    pass
        return call
