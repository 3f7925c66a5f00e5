"""Generation outputs and stream events (core-llm/src/output.rs:5-98)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Union

if TYPE_CHECKING:
    from .tool import ToolCall


@dataclass(frozen=True)
class Usage:
    prompt_tokens: int = 0
    generated_tokens: int = 0

    def total_tokens(self) -> int:
        return self.prompt_tokens + self.generated_tokens


class FinishReason(enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    CANCELLED = "cancelled"
    CONTENT_FILTER = "content_filter"


class Channel(enum.Enum):
    CONTENT = "content"
    THINKING = "thinking"


@dataclass(frozen=True)
class TokenEvent:
    id: int
    text: str
    index: int
    channel: Channel = Channel.CONTENT


@dataclass(frozen=True)
class DoneEvent:
    finish_reason: FinishReason
    usage: Usage


StreamEvent = Union[TokenEvent, DoneEvent]


@dataclass
class TextLlmOutput:
    text: str = ""
    thinking: str | None = None
    tool_calls: list["ToolCall"] = field(default_factory=list)
    usage: Usage = field(default_factory=Usage)
    finish_reason: FinishReason | None = None
