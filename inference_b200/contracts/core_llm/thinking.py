"""Streaming `<think>...</think>` segmentation into content / thinking channels (core-llm/src/thinking.rs:39-135)."""
from __future__ import annotations

from dataclasses import dataclass

from .output import Channel


def max_partial_suffix(pending: str, marker: str) -> int:
    """Length of the longest suffix of `pending` that is a proper-or-full prefix of `marker`."""
    k = min(len(pending), len(marker))
    while k > 0:
        if pending.endswith(marker[:k]):
            return k
        k -= 1
    return 0


@dataclass
class ThinkingSpan:
    channel: Channel
    text: str


class ThinkingSegmenter:
    def __init__(self, open_marker: str = "<think>", close_marker: str = "</think>", start_in_thinking: bool = False):
        assert open_marker and close_marker, "thinking markers must be non-empty"
        self.open, self.close = open_marker, close_marker
        self._in = start_in_thinking
        self.pending = ""

    def in_thinking(self) -> bool:
        return self._in

    def channel(self) -> Channel:
        return Channel.THINKING if self._in else Channel.CONTENT

    def push(self, delta: str) -> list[ThinkingSpan]:
        self.pending += delta
        spans: list[ThinkingSpan] = []
        while True:
            channel = self.channel()
            marker = self.close if self._in else self.open
            pos = self.pending.find(marker)
            if pos >= 0:
                if pos > 0:
                    spans.append(ThinkingSpan(channel, self.pending[:pos]))
                self.pending = self.pending[pos + len(marker):]
                self._in = not self._in
                continue
            hold = max_partial_suffix(self.pending, marker)
            safe = len(self.pending) - hold
            if safe > 0:
                spans.append(ThinkingSpan(channel, self.pending[:safe]))
                self.pending = self.pending[safe:]
            break
        return spans

    def flush(self) -> list[ThinkingSpan]:
        if not self.pending:
            return []
        s = [ThinkingSpan(self.channel(), self.pending)]
        self.pending = ""
        return s
