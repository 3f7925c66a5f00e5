"""Request model: sampling knobs, thinking mode, the generation request and load specs
(core-llm/src/request.rs:10-176)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from .cancel import CancelFlag
from .constraint import Constraint
from .message import Message
from .tool import ToolSpec


@dataclass(frozen=True)
class Sampling:
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 0
    repetition_penalty: float = 1.0
    repetition_context: int = 0

    @staticmethod
    def greedy() -> "Sampling":
        return Sampling(temperature=0.0, top_p=1.0)

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0


class ThinkingMode(enum.Enum):
    AUTO = "auto"
    ENABLED = "enabled"
    DISABLED = "disabled"

    def enable_thinking_kwarg(self) -> bool | None:
        return {ThinkingMode.AUTO: None, ThinkingMode.ENABLED: True, ThinkingMode.DISABLED: False}[self]


@dataclass
class TextLlmRequest:
    messages: list[Message] = field(default_factory=list)
    max_new_tokens: int = 0
    sampling: Sampling = field(default_factory=Sampling)
    seed: int | None = None
    constraint: Constraint | None = None
    thinking: ThinkingMode = ThinkingMode.AUTO
    tools: list[ToolSpec] = field(default_factory=list)
    stop: list[str] = field(default_factory=list)
    cancel: CancelFlag = field(default_factory=CancelFlag)

    def has_image(self) -> bool:
        return any(m.has_image() for m in self.messages)

    def has_video(self) -> bool:
        return any(m.has_video() for m in self.messages)

    def enable_thinking_kwarg(self) -> bool | None:
        return self.thinking.enable_thinking_kwarg()


class Quantize(enum.Enum):
    Q4 = 4
    Q8 = 8


@dataclass
class LoadSpec:
    """Where the weights live (a snapshot directory or a single GGUF file; never a hub id) and whether to
    quantise the projections on load."""
    source: str = ""
    quantize: Quantize | None = None

    @staticmethod
    def dense(source: str) -> "LoadSpec":
        return LoadSpec(source, None)
