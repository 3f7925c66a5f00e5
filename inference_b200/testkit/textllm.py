"""Behavioural conformance suite for any `TextLlm` provider (parity: core-llm-testkit/src/lib.rs:34-680).

`textllm_conformance(make, profile)` runs every check against a fresh provider and raises ConformanceFailure with
the list of violated laws. `StubTextLlm` is a correct weightless provider; its `fault` switch turns it into the
deliberately broken variants that prove each check bites."""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable

from ..contracts.core_llm import (Canceled, CancelFlag, Channel, Constraint, DoneEvent, FinishReason, ImageRef,
                                  InferenceError, InvalidRequest, Message, ModelFormat, PrepareSpec, Role, Sampling,
                                  SnapshotPreparerRegistry, TextLlm, TextLlmCapabilities, TextLlmDescriptor,
                                  TextLlmOutput, TextLlmRequest, ThinkingMode, TokenEvent, ToolSpec, Unsupported,
                                  Usage, VideoRef)
from ..contracts.core_llm.message import Text


class ConformanceFailure(AssertionError):
    pass


@dataclass
class TextLlmProfile:
    prompt: str = "hello"
    max_new_tokens: int = 16
    determinism_seed: int = 7
    determinism_sampling: Sampling = field(default_factory=lambda: Sampling(1.0, 1.0, 0, 1.0, 0))
    image: ImageRef | None = field(default_factory=lambda: ImageRef(8, 8, bytes(8 * 8 * 3)))
    video: VideoRef | None = field(default_factory=lambda: VideoRef(
        (ImageRef(8, 8, bytes(192)), ImageRef(8, 8, bytes([255]) * 192)), (0.0, 0.5)))
    tools: list[ToolSpec] = field(default_factory=lambda: [ToolSpec(
        "get_weather", "Get the current weather for a city",
        {"type": "object", "properties": {"location": {"type": "string"}}, "required": ["location"]})])

    @staticmethod
    def cheap() -> "TextLlmProfile":
        return TextLlmProfile()

    def request(self, sampling: Sampling | None = None, seed: int | None = None) -> TextLlmRequest:
        return TextLlmRequest([Message.user(self.prompt)], self.max_new_tokens, sampling or Sampling.greedy(), seed)


def _collect(p: TextLlm, req: TextLlmRequest):
    events = []
    out = p.generate(req, events.append)
    return out, events


def check_descriptor(p: TextLlm, _profile=None) -> str | None:
    d = p.descriptor()
    if not d.id:
        return "check_descriptor: id is empty"
    if not d.backend:
        return f"check_descriptor[{d.id}]: backend is empty"
    if not d.family:
        return f"check_descriptor[{d.id}]: family is empty"
    return None


def check_validate(p: TextLlm, profile: TextLlmProfile) -> str | None:
    pid = p.descriptor().id
    try:
        p.validate(profile.request())
    except InferenceError as e:
        return f"check_validate[{pid}]: a well-formed request was rejected: {e}"
    bad = [("no messages", TextLlmRequest([], 4)), ("blank content", TextLlmRequest([Message.user("   ")], 4)),
           ("zero budget", TextLlmRequest([Message.user("x")], 0)),
           ("temperature 3", TextLlmRequest([Message.user("x")], 4, Sampling(temperature=3.0))),
           ("top_p 2", TextLlmRequest([Message.user("x")], 4, Sampling(top_p=2.0)))]
    for what, req in bad:
        try:
            p.validate(req)
        except InvalidRequest:
            continue
        except InferenceError as e:
            return f"check_validate[{pid}]: {what} raised {type(e).__name__}, expected InvalidRequest"
        return f"check_validate[{pid}]: {what} was accepted"
    return None


def check_streaming(p: TextLlm, profile: TextLlmProfile) -> str | None:
    pid = p.descriptor().id
    out, events = _collect(p, profile.request())
    toks = [e for e in events if isinstance(e, TokenEvent)]
    dones = [e for e in events if isinstance(e, DoneEvent)]
    if not toks:
        return f"check_streaming[{pid}]: no Token events emitted"
    if len(dones) != 1 or not isinstance(events[-1], DoneEvent):
        return f"check_streaming[{pid}]: expected exactly one Done event, last ({len(dones)} seen)"
    if [e.index for e in toks] != list(range(len(toks))):
        return f"check_streaming[{pid}]: token indices are not 0..n-1"
    content = "".join(e.text for e in toks if e.channel is Channel.CONTENT)
    if content != out.text:
        return f"check_streaming[{pid}]: streamed content {content!r} != output text {out.text!r}"
    if out.finish_reason is None or out.finish_reason is not dones[0].finish_reason:
        return f"check_streaming[{pid}]: finish reason differs between Done event and output"
    if out.usage != dones[0].usage:
        return f"check_streaming[{pid}]: usage differs between Done event and output"
    if out.usage.prompt_tokens == 0:
        return f"check_streaming[{pid}]: usage.prompt_tokens is 0"
    if out.usage.generated_tokens == 0 or out.usage.generated_tokens > profile.max_new_tokens:
        return f"check_streaming[{pid}]: generated_tokens {out.usage.generated_tokens} outside 1..budget"
    return None


def check_cancellation(p: TextLlm, profile: TextLlmProfile) -> str | None:
    pid = p.descriptor().id
    req = profile.request()
    req.cancel.cancel()
    try:
        p.generate(req, lambda e: None)
    except Canceled:
        return None
    except InferenceError as e:
        return f"check_cancellation[{pid}]: pre-cancelled request raised {type(e).__name__}, expected Canceled"
    return f"check_cancellation[{pid}]: pre-cancelled request ran"


def check_mid_stream_cancel(p: TextLlm, profile: TextLlmProfile) -> str | None:
    pid = p.descriptor().id
    req = profile.request()
    seen = []

    def on(e):
        seen.append(e)
        if isinstance(e, TokenEvent) and sum(isinstance(x, TokenEvent) for x in seen) == 1:
            req.cancel.cancel()

    try:
        out = p.generate(req, on)
    except InferenceError as e:
        return f"check_mid_stream_cancel[{pid}]: raised {type(e).__name__}; a mid-stream cancel returns partial output"
    full, _ = _collect(p, profile.request())
    if full.usage.generated_tokens <= 1:
        return None  # the model stops on its own after one token: nothing to cut short
    if out.finish_reason is not FinishReason.CANCELLED:
        return f"check_mid_stream_cancel[{pid}]: finish_reason {out.finish_reason}, expected CANCELLED"
    if out.usage.generated_tokens >= full.usage.generated_tokens:
        return f"check_mid_stream_cancel[{pid}]: cancel did not shorten the generation"
    if not isinstance(seen[-1], DoneEvent):
        return f"check_mid_stream_cancel[{pid}]: no Done event after cancel"
    return None


def check_seed_determinism(p: TextLlm, profile: TextLlmProfile) -> str | None:
    pid = p.descriptor().id
    a, _ = _collect(p, profile.request(profile.determinism_sampling, profile.determinism_seed))
    b, _ = _collect(p, profile.request(profile.determinism_sampling, profile.determinism_seed))
    if a.text != b.text or a.usage != b.usage:
        return f"check_seed_determinism[{pid}]: same seed gave different outputs"
    return None


def _gated(p: TextLlm, req: TextLlmRequest, supported: bool, what: str) -> str | None:
    pid = p.descriptor().id
    if supported:
        try:
            p.validate(req)
        except InferenceError as e:
            return f"check_{what}[{pid}]: advertised but rejected: {e}"
        return None
    try:
        p.validate(req)
    except Unsupported:
        return None
    except InferenceError as e:
        return f"check_{what}[{pid}]: unsupported input raised {type(e).__name__}, expected the typed Unsupported"
    return f"check_{what}[{pid}]: unsupported input was accepted"


def check_multimodal(p: TextLlm, profile: TextLlmProfile) -> str | None:
    if profile.image is None:
        return None
    req = TextLlmRequest([Message(Role.USER, [profile.image, Text(profile.prompt)])], profile.max_new_tokens,
                         Sampling.greedy())
    return _gated(p, req, p.descriptor().capabilities.supports_vision, "multimodal")


def check_video(p: TextLlm, profile: TextLlmProfile) -> str | None:
    if profile.video is None:
        return None
    req = TextLlmRequest([Message(Role.USER, [profile.video, Text(profile.prompt)])], profile.max_new_tokens,
                         Sampling.greedy())
    return _gated(p, req, p.descriptor().capabilities.supports_video, "video")


def check_thinking(p: TextLlm, profile: TextLlmProfile) -> str | None:
    pid = p.descriptor().id
    req = profile.request()
    req.thinking = ThinkingMode.ENABLED
    supported = p.descriptor().capabilities.supports_thinking
    err = _gated(p, req, supported, "thinking")
    if err or not supported:
        return err
    out, events = _collect(p, req)
    think = "".join(e.text for e in events if isinstance(e, TokenEvent) and e.channel is Channel.THINKING)
    if (out.thinking or "") != think:
        return f"check_thinking[{pid}]: streamed reasoning differs from output.thinking"
    if "<think>" in out.text or "</think>" in out.text:
        return f"check_thinking[{pid}]: reasoning markers leaked into the answer text"
    return None


def check_tools(p: TextLlm, profile: TextLlmProfile) -> str | None:
    pid = p.descriptor().id
    req = profile.request()
    req.tools = list(profile.tools)
    supported = p.descriptor().capabilities.supports_tools
    err = _gated(p, req, supported, "tools")
    if err or not supported:
        return err
    out, events = _collect(p, req)
    content = "".join(e.text for e in events if isinstance(e, TokenEvent) and e.channel is Channel.CONTENT)
    if content != out.text:
        return f"check_tools[{pid}]: streamed content does not reconstruct output.text with tools active"
    if "<tool_call>" in out.text:
        return f"check_tools[{pid}]: raw <tool_call> markup leaked into output.text (must be parsed out)"
    for i, c in enumerate(out.tool_calls):
        if not c.name.strip():
            return f"check_tools[{pid}]: parsed tool call #{i} has an empty function name"
    return None


ALL_CHECKS = [check_descriptor, check_validate, check_streaming, check_cancellation, check_mid_stream_cancel,
              check_seed_determinism, check_multimodal, check_video, check_thinking, check_tools]


def textllm_conformance(make: Callable[[], TextLlm], profile: TextLlmProfile | None = None) -> None:
    profile = profile or TextLlmProfile.cheap()
    p = make()
    failures = [msg for chk in ALL_CHECKS if (msg := chk(p, profile))]
    if failures:
        raise ConformanceFailure("\n".join(failures))


def check_snapshot_preparer(registry: SnapshotPreparerRegistry, source: str | Path, out_dir: str | Path,
                            expect_format: ModelFormat) -> str | None:
    rep = registry.prepare_snapshot(PrepareSpec.dense(source, out_dir))
    out = Path(out_dir)
    if rep.input_format is not expect_format:
        return f"check_snapshot_preparer: input_format {rep.input_format}, expected {expect_format}"
    if rep.num_tensors == 0:
        return "check_snapshot_preparer: report counts zero tensors"
    if Path(rep.out_dir) != out or not (out / "config.json").is_file():
        return "check_snapshot_preparer: output directory is not a self-contained snapshot (no config.json)"
    if not any(f.suffix == ".safetensors" for f in out.iterdir()):
        return "check_snapshot_preparer: output directory has no weights"
    return None


# ---- stub providers --------------------------------------------------------------------------------------------
class StubTextLlm(TextLlm):
    """Weightless provider that echoes a deterministic token stream. `fault` selects a deliberate violation:
    no_done, bad_index, ignores_cancel, untyped_cancel, unseeded, accepts_images, accepts_bad_request."""

    def __init__(self, fault: str | None = None):
        self.fault = fault
        self._n = 0
        self._d = TextLlmDescriptor("stub", "stub", "stub", TextLlmCapabilities(
            max_context_tokens=128, max_new_tokens=64, supports_system_prompt=True,
            supported_constraints=[Constraint.JSON]))

    def descriptor(self):
        return self._d

    def validate(self, req):
        if self.fault == "accepts_bad_request":
            return
        if self.fault == "accepts_images":
            img = req.has_image()
            if img:
                return
        self._d.capabilities.validate_request(self._d.id, req)

    def generate(self, req, on_event):
        self.validate(req)
        if req.cancel.is_cancelled():
            if self.fault == "untyped_cancel":
                raise InferenceError("cancelled")
            if self.fault != "ignores_cancel":
                raise Canceled()
        self._n += 1
        seed = (req.seed or 0) if req.sampling.temperature > 0 else 0
        if self.fault == "unseeded" and req.sampling.temperature > 0:
            seed = self._n
        text, n = "", 0
        why = FinishReason.LENGTH
        for i in range(req.max_new_tokens):
            if req.cancel.is_cancelled() and self.fault != "ignores_cancel":
                why = FinishReason.CANCELLED
                break
            piece = f"t{(seed * 31 + i * 7) % 13} "
            text += piece
            on_event(TokenEvent(i, piece, i + 1 if self.fault == "bad_index" else i, Channel.CONTENT))
            n += 1
        usage = Usage(3, n)
        if self.fault != "no_done":
            on_event(DoneEvent(why, usage))
        return TextLlmOutput(text, None, [], usage, why)


BROKEN_FAULTS = ["no_done", "bad_index", "ignores_cancel", "untyped_cancel", "unseeded", "accepts_images",
                 "accepts_bad_request"]
