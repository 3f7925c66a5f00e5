"""Stop strings matched on decoded text, holding back partial matches (core-llm/src/stop.rs:33-96)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class StopChunk:
    emit: str = ""
    stop: bool = False


class StopMatcher:
    def __init__(self, stops):
        self.stops = [s for s in stops if s]
        self.pending = ""

    def is_empty(self) -> bool:
        return not self.stops

    def push(self, delta: str) -> StopChunk:
        if not self.stops:
            return StopChunk(delta, False)
        self.pending += delta
        cut = None
        for s in self.stops:
            pos = self.pending.find(s)
            if pos >= 0:
                cut = pos if cut is None else min(cut, pos)
        if cut is not None:
            emit = self.pending[:cut]
            self.pending = ""
            return StopChunk(emit, True)
        hold = 0
        for s in self.stops:
            k = min(len(self.pending), len(s))
            while k > hold:
                if self.pending.endswith(s[:k]):
                    hold = k
                    break
                k -= 1
        safe = len(self.pending) - hold
        emit = self.pending[:safe]
        self.pending = self.pending[safe:]
        return StopChunk(emit, False)

    def flush(self) -> str:
        p, self.pending = self.pending, ""
        return p
