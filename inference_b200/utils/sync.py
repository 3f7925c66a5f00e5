"""Small synchronisation helpers (candle-gen/src/sync.rs:29-48).

`lock_recover` takes a lock even when a previous holder died with an exception (Python locks do not poison, the
helper exists so call sites read the same as the reference's and to give a timeout-free context manager);
`cached` fills a one-slot cache under its lock so concurrent first uses load once."""
from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import Callable, Generic, TypeVar

T = TypeVar("T")


@contextmanager
def lock_recover(lock: threading.Lock):
    lock.acquire()
    try:
        yield
    finally:
        lock.release()


class Slot(Generic[T]):
    """A lock plus an optional value."""

    def __init__(self) -> None:
        self.lock = threading.Lock()
        self.value: T | None = None


def cached(slot: "Slot[T]", load: Callable[[], T]) -> T:
    """The slot's value, loading it on first use. A load that raises leaves the slot empty so the next call retries."""
    with lock_recover(slot.lock):
        if slot.value is None:
            slot.value = load()
        return slot.value
