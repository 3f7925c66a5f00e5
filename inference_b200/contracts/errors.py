"""Typed errors of the provider contracts.

`Canceled` and `Unsupported` must stay typed end to end so callers can distinguish a user cancel or a
capability gap from a backend failure (core-llm/src/error.rs:11-40; gen-core mirrors the same set).
"""
from __future__ import annotations


class InferenceError(Exception):
    """Base of every error raised through the contracts."""

    kind = "msg"


class BackendError(InferenceError):
    kind = "backend"


class LoadError(InferenceError):
    kind = "load"


class InvalidRequest(InferenceError):
    kind = "invalid_request"


class Unsupported(InferenceError):
    kind = "unsupported"


class Canceled(InferenceError):
    kind = "canceled"

    def __init__(self, msg: str = "canceled"):
        super().__init__(msg)


class IoError(InferenceError):
    kind = "io"


class ConfigError(LoadError):
    kind = "load"


class CollectiveTimeout(BackendError):
    """A bounded device-side wait on a peer flag ran out of budget."""
