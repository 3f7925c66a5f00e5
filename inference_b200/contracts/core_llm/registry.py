"""Explicit, immutable text-LLM registry with model-first selection (core-llm/src/registry.rs:25-241).

No global state and no import-time discovery: a runtime bundle builds a registry from registrations it
names. `load_for_model` probes each registration's weightless `can_load(spec)` (reads config.json / a
GGUF header only), filters by the capabilities the request surface needs, and prefers a text provider
over a vision one when vision was not asked for."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterable

from ..errors import InferenceError, Unsupported
from .capabilities import TextLlmDescriptor
from .constraint import Constraint
from .request import LoadSpec, TextLlmRequest
from .text_llm import TextLlm


@dataclass(frozen=True)
class TextLlmRegistration:
    descriptor: Callable[[], TextLlmDescriptor]
    load: Callable[[LoadSpec], TextLlm]
    can_load: Callable[[LoadSpec], bool]
    weightless_vision: Callable[[LoadSpec], bool] | None = None


@dataclass
class ModelRequirements:
    vision: bool = False
    video: bool = False
    constraints: list[Constraint] = field(default_factory=list)

    @staticmethod
    def from_request(req: TextLlmRequest) -> "ModelRequirements":
        video = req.has_video()
        return ModelRequirements(req.has_image() or video, video, [req.constraint] if req.constraint else [])

    def with_vision(self) -> "ModelRequirements":
        self.vision = True
        return self

    def with_video(self) -> "ModelRequirements":
        self.video = self.vision = True
        return self

    def with_constraint(self, c: Constraint) -> "ModelRequirements":
        if c not in self.constraints:
            self.constraints.append(c)
        return self


class TextLlmRegistryBuilder:
    def __init__(self):
        self._regs: list[TextLlmRegistration] = []

    def register(self, reg: TextLlmRegistration) -> "TextLlmRegistryBuilder":
        self._regs.append(reg)
        return self

    def extend(self, regs: Iterable[TextLlmRegistration]) -> "TextLlmRegistryBuilder":
        self._regs.extend(regs)
        return self

    def build(self) -> "TextLlmRegistry":
        seen = set()
        for r in self._regs:
            i = r.descriptor().id
            if i in seen:
                raise InferenceError(f"duplicate textllm id '{i}' in explicit registry")
            seen.add(i)
        return TextLlmRegistry(tuple(self._regs))


def _serves_vision(reg: TextLlmRegistration, spec: LoadSpec) -> bool:
    return bool(reg.weightless_vision and reg.weightless_vision(spec)) or reg.descriptor().capabilities.supports_vision


def _summary(regs) -> str:
    if not regs:
        return "(none)"
    return ", ".join(sorted({f"{r.descriptor().id} ({r.descriptor().backend})" for r in regs}))


def _raw_arch_hint(spec: LoadSpec) -> str | None:
    p = Path(spec.source)
    cfg = p / "config.json" if p.is_dir() else p
    try:
        v = json.loads(cfg.read_text())
    except Exception:
        return None
    parts = []
    a = v.get("architectures")
    if isinstance(a, list) and a and isinstance(a[0], str):
        parts.append(f"architectures={a[0]}")
    if isinstance(v.get("model_type"), str):
        parts.append(f"model_type={v['model_type']}")
    tc = v.get("text_config")
    if isinstance(tc, dict) and isinstance(tc.get("model_type"), str):
        parts.append(f"text_config.model_type={tc['model_type']}")
    return ", ".join(parts) if parts else None


class TextLlmRegistry:
    def __init__(self, regs: tuple[TextLlmRegistration, ...]):
        self._regs = regs

    def registrations(self) -> tuple[TextLlmRegistration, ...]:
        return self._regs

    def find(self, provider_id: str) -> TextLlmRegistration | None:
        for r in self._regs:
            if r.descriptor().id == provider_id:
                return r
        return None

    def load_textllm(self, provider_id: str, spec: LoadSpec) -> TextLlm:
        r = self.find(provider_id)
        if r is None:
            raise InferenceError(f"no textllm registered for id '{provider_id}'")
        return r.load(spec)

    def select(self, spec: LoadSpec, reqs: ModelRequirements | None = None) -> TextLlmRegistration:
        reqs = reqs or ModelRequirements()
        accepting = [r for r in self._regs if r.can_load(spec)]
        if not accepting:
            hint = _raw_arch_hint(spec)
            arch = f" ({hint})" if hint else ""
            raise Unsupported(f"no registered provider can serve model '{spec.source}'{arch}; "
                              f"available providers: {_summary(self._regs)}")

        def meets(r: TextLlmRegistration) -> bool:
            if reqs.vision and not _serves_vision(r, spec):
                return False
            caps = r.descriptor().capabilities
            return all(caps.supports_constraint(c) for c in reqs.constraints)

        viable = [r for r in accepting if meets(r)]
        if not viable:
            raise Unsupported(
                f"model '{spec.source}' is loadable, but no available provider meets the requested capabilities "
                f"(vision={reqs.vision}, constraints={[c.name for c in reqs.constraints]}); providers that match "
                f"the architecture: {_summary(accepting)}")
        if len(viable) > 1 and not reqs.vision:
            for r in viable:
                if not _serves_vision(r, spec):
                    return r
        return viable[0]

    def load_for_model(self, spec: LoadSpec) -> TextLlm:
        return self.load_for_model_with(spec, ModelRequirements())

    def load_for_model_with(self, spec: LoadSpec, reqs: ModelRequirements) -> TextLlm:
        return self.select(spec, reqs).load(spec)
