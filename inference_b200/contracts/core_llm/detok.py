"""Incremental detokenisation that never emits a transient U+FFFD (core-llm/src/detok.rs:45-62).

Feed the full decoded text so far; a trailing run of replacement characters (an incomplete multi-byte
sequence) is held back until it resolves."""
from __future__ import annotations


class IncrementalDetok:
    def __init__(self):
        self.shown = 0

    def push(self, decoded: str) -> str | None:
        stable = decoded.rstrip("�")
        if len(stable) <= self.shown:
            return None
        delta = stable[self.shown:]
        self.shown = len(stable)
        return delta
