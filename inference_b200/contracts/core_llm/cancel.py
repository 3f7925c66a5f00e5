"""Cooperative cancellation flag carried in-band on a request (core-llm/src/cancel.rs:1-37).

A request that arrives already cancelled fails with `Canceled` before inference starts; a flag set mid
stream ends the generation with partial output and FinishReason.CANCELLED."""
from __future__ import annotations

import threading


class CancelFlag:
    def __init__(self):
        self._ev = threading.Event()

    def cancel(self) -> None:
        self._ev.set()

    def is_cancelled(self) -> bool:
        return self._ev.is_set()

    def __repr__(self) -> str:
        return f"CancelFlag(cancelled={self.is_cancelled()})"
