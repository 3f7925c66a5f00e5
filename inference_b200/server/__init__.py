"""OpenAI-compatible serving front end."""
from .http import LlmService, serve, serve_in_thread  # noqa: F401
