"""Metrics, structured logging and tracing helpers."""
from . import logging, metrics, tracing  # noqa: F401
