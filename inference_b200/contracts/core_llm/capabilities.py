"""Provider capabilities, the shared request-validation floor and descriptors
(core-llm/src/capabilities.rs:9-137)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import InvalidRequest, Unsupported
from .constraint import Constraint
from .message import Role
from .request import TextLlmRequest, ThinkingMode


@dataclass
class TextLlmCapabilities:
    max_context_tokens: int = 0
    max_new_tokens: int = 0
    supports_system_prompt: bool = False
    supports_vision: bool = False
    supports_video: bool = False
    supports_thinking: bool = False
    supports_tools: bool = False
    supported_constraints: list[Constraint] = field(default_factory=list)

    def supports_constraint(self, c: Constraint) -> bool:
        return c in self.supported_constraints

    def validate_request(self, provider_id: str, req: TextLlmRequest) -> None:
        """Raises InvalidRequest for malformed requests and the typed Unsupported for capability gaps."""
        def reject(msg: str):
            raise InvalidRequest(f"[{provider_id}] {msg}")

        if not req.messages:
            reject("request has no messages")
        if all(not m.text_content().strip() and not m.has_image() and not m.has_video() for m in req.messages):
            reject("request has no non-empty content")
        if not self.supports_system_prompt and any(m.role is Role.SYSTEM for m in req.messages):
            raise Unsupported(f"[{provider_id}] provider does not support a system prompt")
        if not self.supports_vision and req.has_image():
            raise Unsupported(f"[{provider_id}] provider does not support image (vision) input")
        if not self.supports_video and req.has_video():
            raise Unsupported(f"[{provider_id}] provider does not support video input")
        if not self.supports_thinking and req.thinking is ThinkingMode.ENABLED:
            raise Unsupported(f"[{provider_id}] provider does not support a thinking (reasoning) mode")
        if not self.supports_tools and req.tools:
            raise Unsupported(f"[{provider_id}] provider does not support tool (function) calling")
        if req.constraint is not None and not self.supports_constraint(req.constraint):
            raise Unsupported(f"[{provider_id}] provider does not support the {req.constraint.name} constraint")
        s = req.sampling
        if not (0.0 <= s.temperature <= 2.0):
            reject(f"temperature {s.temperature} out of [0, 2]")
        if not (0.0 <= s.top_p <= 1.0):
            reject(f"top_p {s.top_p} out of [0, 1]")
        if req.max_new_tokens == 0:
            reject("max_new_tokens must be >= 1")
        if self.max_new_tokens > 0 and req.max_new_tokens > self.max_new_tokens:
            reject(f"max_new_tokens {req.max_new_tokens} exceeds cap {self.max_new_tokens}")


@dataclass
class TextLlmDescriptor:
    id: str
    family: str
    backend: str
    capabilities: TextLlmCapabilities
