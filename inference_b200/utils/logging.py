"""Structured logging: one JSON object per line on stderr, level from SWB_LOG (error|warn|info|debug, default warn).
Mirrors the role of the reference's `tracing` subscriber set-up in its binaries."""
from __future__ import annotations

import json
import os
import sys
import threading
import time

_LEVELS = {"error": 40, "warn": 30, "info": 20, "debug": 10}
_lock = threading.Lock()


def _threshold() -> int:
    return _LEVELS.get(os.environ.get("SWB_LOG", "warn").lower(), 30)


def log(level: str, event: str, **fields) -> None:
    if _LEVELS.get(level, 20) < _threshold():
        return
    rec = {"ts": round(time.time(), 3), "level": level, "event": event, **fields}
    with _lock:
        sys.stderr.write(json.dumps(rec, default=str) + "\n")
        sys.stderr.flush()


def info(event: str, **f) -> None:
    log("info", event, **f)


def warn(event: str, **f) -> None:
    log("warn", event, **f)


def error(event: str, **f) -> None:
    log("error", event, **f)


def debug(event: str, **f) -> None:
    log("debug", event, **f)
