"""Chat messages with text / image / video content blocks (core-llm/src/message.rs:10-200)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Union

if TYPE_CHECKING:
    from .tool import ToolCall


class Role(enum.Enum):
    SYSTEM = "system"
    USER = "user"
    ASSISTANT = "assistant"
    TOOL = "tool"

    def as_str(self) -> str:
        return self.value


@dataclass(frozen=True)
class ImageRef:
    """Raw RGB8 pixels, row-major, exactly width * height * 3 bytes."""
    width: int
    height: int
    pixels: bytes

    def __post_init__(self):
        expected = self.width * self.height * 3
        if len(self.pixels) != expected:
            raise ValueError(f"ImageRef: {self.width}x{self.height} needs {expected} RGB bytes, got {len(self.pixels)}")


@dataclass(frozen=True)
class VideoRef:
    frames: tuple[ImageRef, ...]
    timestamps: tuple[float, ...]

    def __post_init__(self):
        if not self.frames:
            raise ValueError("VideoRef: needs at least one frame")
        if len(self.frames) != len(self.timestamps):
            raise ValueError(f"VideoRef: {len(self.frames)} frames but {len(self.timestamps)} timestamps "
                             "(need one timestamp per frame)")

    def __len__(self) -> int:
        return len(self.frames)


@dataclass(frozen=True)
class Text:
    text: str


Content = Union[Text, ImageRef, VideoRef]


@dataclass
class Message:
    role: Role
    content: list[Content]
    thinking: str | None = None
    tool_calls: list["ToolCall"] = field(default_factory=list)

    @staticmethod
    def text(role: Role, text: str) -> "Message":
        return Message(role, [Text(text)])

    @staticmethod
    def system(text: str) -> "Message":
        return Message.text(Role.SYSTEM, text)

    @staticmethod
    def user(text: str) -> "Message":
        return Message.text(Role.USER, text)

    @staticmethod
    def assistant(text: str) -> "Message":
        return Message.text(Role.ASSISTANT, text)

    def with_thinking(self, thinking: str) -> "Message":
        self.thinking = thinking
        return self

    def with_tool_calls(self, calls: list["ToolCall"]) -> "Message":
        self.tool_calls = list(calls)
        return self

    def text_content(self) -> str:
        """Concatenated text blocks; image and video blocks are omitted."""
        return "".join(c.text for c in self.content if isinstance(c, Text))

    def has_image(self) -> bool:
        return any(isinstance(c, ImageRef) for c in self.content)

    def has_video(self) -> bool:
        return any(isinstance(c, VideoRef) for c in self.content)
