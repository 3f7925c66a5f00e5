"""The streaming, cancellable text-LLM provider contract (core-llm/src/text_llm.rs:17-38)."""
from __future__ import annotations

import abc
from typing import Callable

from .capabilities import TextLlmDescriptor
from .output import StreamEvent, TextLlmOutput
from .request import TextLlmRequest


class TextLlm(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> TextLlmDescriptor: ...

    @abc.abstractmethod
    def validate(self, req: TextLlmRequest) -> None:
        """Raise InvalidRequest / Unsupported without touching the model."""

    @abc.abstractmethod
    def generate(self, req: TextLlmRequest, on_event: Callable[[StreamEvent], None]) -> TextLlmOutput:
        """Stream TokenEvents then exactly one DoneEvent; returns the assembled output."""

    def complete(self, req: TextLlmRequest) -> TextLlmOutput:
        return self.generate(req, lambda _e: None)
