"""Conformance suite for `Generator` providers (parity: gen-core-testkit/src/lib.rs:131-231,307-720).

Each check returns None on success and raises `ConformanceFailure` with a labelled message otherwise. `conformance`
runs the model-level laws (validate honesty, exact progress, progress contract, cancellation, pre-cancellation, seed
determinism); `registry_conformance` runs the weight-free registry laws (descriptor round trip, component load
gate). The suite renders the cheap profile about five times."""
from __future__ import annotations

import copy
from dataclasses import dataclass, replace

from ..contracts.errors import Canceled, InferenceError
from ..contracts.gen_core.generator import (Conditioning, ConditioningKind, GenerationOutput, GenerationRequest,
                                            Generator)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import ProviderRegistry
from ..contracts.gen_core.runtime import CancelFlag, LoadSpec, ProgressDecoding, ProgressStep, WeightsSource


class ConformanceFailure(AssertionError):
    pass


@dataclass
class Profile:
    prompt: str = "a fox"
    width: int = 256
    height: int = 256
    steps: int = 2          # requested AND expected resolved step count
    seed: int = 42
    cancel_steps: int = 6
    conditioning: tuple = ()      # conditioning every request of the profile carries (image -> video providers ...)


def base_request(p: Profile) -> GenerationRequest:
    return GenerationRequest(prompt=p.prompt, width=p.width, height=p.height, steps=p.steps, seed=p.seed,
                             conditioning=list(p.conditioning))


def output_bytes(out: GenerationOutput) -> bytes:
    if out.images:
        return b"".join(i.pixels for i in out.images)
    if out.video_frames:
        return b"".join(f.pixels for f in out.video_frames)
    if out.audio is not None:
        import struct

        return struct.pack(f"<{len(out.audio.samples)}f", *out.audio.samples)
    return b""


def _blank(p: Profile) -> Image:
    return Image(p.width, p.height, bytes(p.width * p.height * 3))


def _fresh(req: GenerationRequest, **kw) -> GenerationRequest:
    r = copy.copy(req)
    r.cancel = CancelFlag()
    for k, v in kw.items():
        setattr(r, k, v)
    return r


def _rejects(g: Generator, req: GenerationRequest) -> bool:
    try:
        g.validate(req)
    except InferenceError:
        return True
    return False


def check_validate_honesty(g: Generator, p: Profile) -> None:
    d = g.descriptor()
    caps, mid = d.capabilities, d.id
    req = base_request(p)
    try:
        g.validate(req)
    except InferenceError as e:
        raise ConformanceFailure(f"validate-honesty[{mid}]: the in-capability cheap request was rejected: {e}")
    for s in caps.samplers:
        if _rejects(g, _fresh(req, sampler=s)):
            raise ConformanceFailure(f"validate-honesty[{mid}]: advertised sampler {s!r} was rejected by validate()")
    for s in caps.schedulers:
        if _rejects(g, _fresh(req, scheduler=s)):
            raise ConformanceFailure(f"validate-honesty[{mid}]: advertised scheduler {s!r} was rejected")
    if caps.max_size:
        big = caps.max_size + 64
        if not _rejects(g, _fresh(req, width=big, height=big)):
            raise ConformanceFailure(f"validate-honesty[{mid}]: a {big}x{big} request (above max_size "
                                     f"{caps.max_size}) was accepted by validate()")
    if not _rejects(g, _fresh(req, count=caps.max_count + 1)):
        raise ConformanceFailure(f"validate-honesty[{mid}]: count above max_count {caps.max_count} was accepted")
    for kind in (ConditioningKind.MASK, ConditioningKind.DEPTH, ConditioningKind.REFERENCE):
        if not caps.accepts(kind):
            if not _rejects(g, _fresh(req, conditioning=[Conditioning(kind=kind, image=_blank(p))])):
                raise ConformanceFailure(f"validate-honesty[{mid}]: undeclared {kind.name} conditioning was accepted")
            break
    if not caps.supports_negative_prompt and not _rejects(g, _fresh(req, negative_prompt="blurry")):
        raise ConformanceFailure(f"validate-honesty[{mid}]: negative prompt accepted but not advertised")
    if not caps.supports_guidance and not _rejects(g, _fresh(req, guidance=3.5)):
        raise ConformanceFailure(f"validate-honesty[{mid}]: guidance accepted but not advertised")


def _run(g: Generator, req: GenerationRequest):
    events = []
    out = g.generate(req, events.append)
    return out, events


def check_progress(g: Generator, p: Profile) -> None:
    mid = g.descriptor().id
    _, events = _run(g, base_request(p))
    steps = [(e.current, e.total) for e in events if isinstance(e, ProgressStep)]
    if not steps:
        raise ConformanceFailure(f"progress[{mid}]: generate() emitted no step events")
    total = steps[0][1]
    if any(t != total for _, t in steps):
        raise ConformanceFailure(f"progress[{mid}]: Step.total changed mid-run: {steps}")
    if [c for c, _ in steps] != list(range(1, total + 1)):
        raise ConformanceFailure(f"progress[{mid}]: Step.current must be exactly 1..={total}; got {steps}")
    if total != p.steps:
        raise ConformanceFailure(f"progress[{mid}]: Step.total ({total}) != the expected step count ({p.steps})")


def check_progress_contract(g: Generator, p: Profile) -> None:
    mid = g.descriptor().id
    _, events = _run(g, base_request(p))
    steps = [(e.current, e.total) for e in events if isinstance(e, ProgressStep)]
    if not steps or steps[0][1] == 0:
        raise ConformanceFailure(f"progress-contract[{mid}]: no step events or total 0")
    total, prev = steps[0][1], 0
    for c, t in steps:
        if t != total or c > total or c < prev:
            raise ConformanceFailure(f"progress-contract[{mid}]: bad step sequence {steps}")
        prev = c
    if prev != total:
        raise ConformanceFailure(f"progress-contract[{mid}]: the bar stopped at {prev} of {total}")
    n_dec = sum(isinstance(e, ProgressDecoding) for e in events)
    if n_dec != 1:
        raise ConformanceFailure(f"progress-contract[{mid}]: Decoding emitted {n_dec} times, expected exactly 1")


def check_cancellation(g: Generator, p: Profile) -> None:
    mid = g.descriptor().id
    req = replace(base_request(p), steps=p.cancel_steps, cancel=CancelFlag())
    seen = {"steps": 0, "after": 0}

    def on_progress(e):
        if isinstance(e, ProgressStep):
            seen["steps"] += 1
            if req.cancel.is_cancelled():
                seen["after"] += 1
            req.cancel.cancel()

    try:
        g.generate(req, on_progress)
    except Canceled:
        if seen["steps"] == 0:
            raise ConformanceFailure(f"cancellation[{mid}]: no step was emitted, cancellation was not exercised")
        if seen["after"] > 2:
            raise ConformanceFailure(f"cancellation[{mid}]: {seen['after']} further steps after the cancel trip")
        return
    except InferenceError as e:
        raise ConformanceFailure(f"cancellation[{mid}]: must raise the typed Canceled, got {type(e).__name__}: {e}")
    raise ConformanceFailure(f"cancellation[{mid}]: generate() ran to completion despite the cancel flag")


def check_pre_cancellation(g: Generator, p: Profile) -> None:
    mid = g.descriptor().id
    req = base_request(p)
    req.cancel.cancel()
    events = []
    try:
        g.generate(req, events.append)
    except Canceled:
        if any(isinstance(e, ProgressStep) for e in events):
            raise ConformanceFailure(f"pre-cancellation[{mid}]: steps ran although the flag was set before the call")
        return
    raise ConformanceFailure(f"pre-cancellation[{mid}]: a request cancelled before the call must raise Canceled")


def check_seed_determinism(g: Generator, p: Profile) -> None:
    mid = g.descriptor().id
    a, _ = _run(g, base_request(p))
    b, _ = _run(g, base_request(p))
    if output_bytes(a) != output_bytes(b):
        raise ConformanceFailure(f"seed-determinism[{mid}]: the same seed gave different outputs")
    c, _ = _run(g, replace(base_request(p), seed=p.seed + 1, cancel=CancelFlag()))
    if output_bytes(a) == output_bytes(c):
        raise ConformanceFailure(f"seed-determinism[{mid}]: a different seed gave identical outputs")


def check_batch_seed_law(g: Generator, p: Profile) -> None:
    """Image i of a count-n request equals a count-1 request at seed + i."""
    mid = g.descriptor().id
    if g.descriptor().capabilities.max_count < 2:
        return
    both, _ = _run(g, replace(base_request(p), count=2, cancel=CancelFlag()))
    second, _ = _run(g, replace(base_request(p), seed=p.seed + 1, cancel=CancelFlag()))
    if len(both.images) != 2 or both.images[1].pixels != second.images[0].pixels:
        raise ConformanceFailure(f"batch-seed[{mid}]: image 1 of a batch must equal a single render at seed + 1")


def conformance(g: Generator, p: Profile | None = None) -> None:
    p = p or Profile()
    check_validate_honesty(g, p)
    check_progress(g, p)
    check_progress_contract(g, p)
    check_cancellation(g, p)
    check_pre_cancellation(g, p)
    check_seed_determinism(g, p)


def registry_conformance(reg: ProviderRegistry, provider_id: str, spec: LoadSpec) -> None:
    """Weight-free laws: the registry knows the id, its descriptor passes the structural checks, the loaded
    provider's descriptor equals the registered one, and a spec naming an unknown component is refused."""
    r = reg.find("generator", provider_id)
    if r is None:
        raise ConformanceFailure(f"registry[{provider_id}]: not registered")
    errs = [e for e in reg.descriptor_conformance_errors() if provider_id in e]
    if errs:
        raise ConformanceFailure(f"registry[{provider_id}]: descriptor errors: {errs}")
    g = reg.load(provider_id, spec)
    d0, d1 = r.descriptor(), g.descriptor()
    if (d0.id, d0.family, d0.backend, d0.modality) != (d1.id, d1.family, d1.backend, d1.modality) or \
            d0.capabilities != d1.capabilities:
        raise ConformanceFailure(f"registry[{provider_id}]: loaded descriptor differs from the registered one")
    if not d0.required_components:
        bad = copy.copy(spec)
        bad.components = {"no_such_component": WeightsSource.dir("/nonexistent")}
        try:
            reg.load(provider_id, bad)
        except InferenceError:
            return
        raise ConformanceFailure(f"registry[{provider_id}]: a spec with an undeclared component was accepted")
