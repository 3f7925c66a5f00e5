"""Chat templates: built-in Llama-3 and ChatML layouts and Jinja templates read from a tokenizer_config.json
(core-llm/src/template.rs:23-330). The Jinja environment mirrors what `transformers` uses (immutable sandbox,
trim/lstrip blocks, `raise_exception`, `strftime_now`); `enable_thinking` and `tools` are omitted from the
render context when not provided so `is defined` / truthiness tests in templates behave."""
from __future__ import annotations

import abc
import json
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..errors import InferenceError
from .message import Message
from .tool import ToolSpec


@dataclass
class RenderOptions:
    add_generation_prompt: bool = False
    enable_thinking: bool | None = None
    tools: list[ToolSpec] = field(default_factory=list)

    @staticmethod
    def generation() -> "RenderOptions":
        return RenderOptions(add_generation_prompt=True)

    def with_enable_thinking(self, v: bool | None) -> "RenderOptions":
        self.enable_thinking = v
        return self

    def with_tools(self, tools: list[ToolSpec]) -> "RenderOptions":
        self.tools = list(tools)
        return self


class ChatTemplate(abc.ABC):
    @abc.abstractmethod
    def render(self, messages: list[Message], add_generation_prompt: bool) -> str: ...

    def render_with(self, messages: list[Message], opts: RenderOptions) -> str:
        return self.render(messages, opts.add_generation_prompt)


class Llama3Template(ChatTemplate):
    def render(self, messages, add_generation_prompt):
        out = ["<|begin_of_text|>"]
        for m in messages:
            out.append(f"<|start_header_id|>{m.role.as_str()}<|end_header_id|>\n\n{m.text_content()}<|eot_id|>")
        if add_generation_prompt:
            out.append("<|start_header_id|>assistant<|end_header_id|>\n\n")
        return "".join(out)


class ChatMlTemplate(ChatTemplate):
    def render(self, messages, add_generation_prompt):
        out = [f"<|im_start|>{m.role.as_str()}\n{m.text_content()}<|im_end|>\n" for m in messages]
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n")
        return "".join(out)


def _extract_chat_template(config: dict[str, Any]) -> str | None:
    ct = config.get("chat_template")
    if isinstance(ct, str):
        return ct
    if isinstance(ct, list) and ct:
        pick = next((e for e in ct if isinstance(e, dict) and e.get("name") == "default"), ct[0])
        t = pick.get("template") if isinstance(pick, dict) else None
        return t if isinstance(t, str) else None
    return None


def _extract_token(v: Any) -> str | None:
    if isinstance(v, str):
        return v
    if isinstance(v, dict) and isinstance(v.get("content"), str):
        return v["content"]
    return None


class JinjaChatTemplate(ChatTemplate):
    def __init__(self, source: str, bos_token: str = "", eos_token: str = ""):
        self.source, self.bos_token, self.eos_token = source, bos_token, eos_token
        self.template_error: str | None = None
        self._template = None
        try:
            from jinja2.sandbox import ImmutableSandboxedEnvironment

            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)

            def raise_exception(msg):
                raise InferenceError(f"chat template render: {msg}")

            env.globals["raise_exception"] = raise_exception
            env.globals["strftime_now"] = lambda fmt: time.strftime(fmt, time.gmtime())
            env.filters["tojson"] = lambda v, indent=None: json.dumps(v, ensure_ascii=False, indent=indent)
            self._template = env.from_string(source)
        except InferenceError:
            raise
        except Exception as e:  # a broken template surfaces at render time, like the reference
            self.template_error = f"chat template render: {e}"

    @staticmethod
    def from_tokenizer_config(config: dict[str, Any]) -> "JinjaChatTemplate":
        src = _extract_chat_template(config)
        if src is None:
            raise InferenceError("tokenizer_config.json has no chat_template")
        return JinjaChatTemplate(src, _extract_token(config.get("bos_token")) or "",
                                 _extract_token(config.get("eos_token")) or "")

    @staticmethod
    def from_tokenizer_config_file(path: str | Path) -> "JinjaChatTemplate":
        try:
            cfg = json.loads(Path(path).read_text())
        except json.JSONDecodeError as e:
            raise InferenceError(f"parse tokenizer_config.json: {e}") from e
        return JinjaChatTemplate.from_tokenizer_config(cfg)

    def render(self, messages, add_generation_prompt):
        return self.render_with(messages, RenderOptions(add_generation_prompt=add_generation_prompt))

    def render_with(self, messages, opts):
        if self.template_error:
            raise InferenceError(self.template_error)
        msgs = []
        for m in messages:
            d: dict[str, Any] = {"role": m.role.as_str(), "content": m.text_content()}
            if m.thinking is not None:
                d["reasoning_content"] = m.thinking
                d["thinking"] = m.thinking
            if m.tool_calls:
                d["tool_calls"] = [c.to_template_json() for c in m.tool_calls]
            msgs.append(d)
        ctx: dict[str, Any] = {"messages": msgs, "add_generation_prompt": opts.add_generation_prompt,
                               "bos_token": self.bos_token, "eos_token": self.eos_token}
        if opts.enable_thinking is not None:
            ctx["enable_thinking"] = opts.enable_thinking
        if opts.tools:
            ctx["tools"] = [t.to_template_json() for t in opts.tools]
        try:
            return self._template.render(**ctx)
        except InferenceError:
            raise
        except Exception as e:
            raise InferenceError(f"chat template render: {e}") from e
