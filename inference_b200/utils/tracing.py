"""Span timing for host code and CUDA-event timing for device work; spans nest per thread and are exported as a
Chrome-trace JSON (the reference's tracing story is `tracing` spans plus per-stage timers in its bench harnesses)."""
from __future__ import annotations

import json
import threading
import time
from contextlib import contextmanager

_local = threading.local()
_events: list[dict] = []
_lock = threading.Lock()
enabled = False


def enable(on: bool = True) -> None:
    global enabled
    enabled = on


@contextmanager
def span(name: str, **args):
    if not enabled:
        yield
        return
    t0 = time.perf_counter_ns()
    try:
        yield
    finally:
        t1 = time.perf_counter_ns()
        with _lock:
            _events.append({"name": name, "ph": "X", "ts": t0 / 1e3, "dur": (t1 - t0) / 1e3, "pid": 0,
                            "tid": threading.get_ident() % 100000, "args": args})


class DeviceTimer:
    """CUDA-event stopwatch on the current stream: `with DeviceTimer() as t: ...; t.ms` (synchronises on exit)."""

    def __enter__(self):
        import torch

        self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._e0.record()
        return self

    def __exit__(self, *exc):
        import torch

        self._e1.record()
        torch.cuda.synchronize()
        self.ms = self._e0.elapsed_time(self._e1)


def export_chrome_trace(path: str) -> int:
    with _lock:
        ev = list(_events)
    with open(path, "w") as f:
        json.dump({"traceEvents": ev}, f)
    return len(ev)


def clear() -> None:
    with _lock:
        _events.clear()
