"""Conformance suite for audio generators (gen-core-testkit/src/audio_generator.rs:110-1082, the laws that apply to a
text-to-speech / text-to-audio provider): descriptor shape, validate honesty for every advertised and unadvertised
audio knob, output invariants, exact progress, typed cancellation, seed determinism, target-duration behaviour."""
from __future__ import annotations

import math
from dataclasses import dataclass

from ..contracts.errors import Canceled, InferenceError
from ..contracts.gen_core.generator import AudioParams, GenerationRequest, Generator, Modality
from ..contracts.gen_core.runtime import CancelFlag, ProgressStep
from .generator import ConformanceFailure


@dataclass
class AudioProfile:
    prompt: str = "hello world"
    seed: int = 7
    voice: str | None = None
    target_duration: float | None = None     # when set, the duration law is checked against it
    duration_tolerance: float = 0.5          # relative


def _req(p: AudioProfile, **audio) -> GenerationRequest:
    a = AudioParams(voice=p.voice)
    for k, v in audio.items():
        setattr(a, k, v)
    return GenerationRequest(prompt=p.prompt, seed=p.seed, audio=a)


def _rejects(g: Generator, req: GenerationRequest) -> bool:
    try:
        g.validate(req)
    except InferenceError:
        return True
    return False


def audio_conformance(g: Generator, p: AudioProfile | None = None) -> None:
    p = p or AudioProfile()
    d = g.descriptor()
    caps, mid = d.capabilities, d.id
    if d.modality is not Modality.AUDIO:
        raise ConformanceFailure(f"{mid}: an audio generator must declare Modality.AUDIO")
    if not caps.audio_sample_rates:
        raise ConformanceFailure(f"{mid}: no audio_sample_rates advertised")
    # ---- validate honesty ----
    if _rejects(g, _req(p)):
        raise ConformanceFailure(f"{mid}: the plain in-capability request was rejected")
    if not _rejects(g, GenerationRequest(prompt="  ", seed=p.seed, audio=AudioParams())):
        raise ConformanceFailure(f"{mid}: a blank script was accepted")
    for v in caps.audio_voices:
        if _rejects(g, _req(p, voice=v)):
            raise ConformanceFailure(f"{mid}: advertised voice {v!r} rejected by validate()")
    for lang in caps.audio_languages:
        if _rejects(g, _req(p, language=lang)):
            raise ConformanceFailure(f"{mid}: advertised language {lang!r} rejected")
    for sr in caps.audio_sample_rates:
        if _rejects(g, _req(p, sample_rate=sr)):
            raise ConformanceFailure(f"{mid}: advertised sample rate {sr} rejected")
    if caps.audio_voices and not _rejects(g, _req(p, voice="no_such_voice_")):
        raise ConformanceFailure(f"{mid}: an unadvertised voice was accepted")
    if not _rejects(g, _req(p, sample_rate=12_345)):
        raise ConformanceFailure(f"{mid}: an unadvertised sample rate was accepted")
    if caps.audio_languages and not _rejects(g, _req(p, language="xx-none")):
        raise ConformanceFailure(f"{mid}: an unadvertised language was accepted")
    if caps.max_audio_duration_secs is not None and not _rejects(g, _req(p, target_duration=caps.max_audio_duration_secs * 2)):
        raise ConformanceFailure(f"{mid}: a target duration above the advertised maximum was accepted")
    if not _rejects(g, _req(p, target_duration=float("nan"))):
        raise ConformanceFailure(f"{mid}: a NaN target duration was accepted")
    if not caps.supports_multi_speaker and not _rejects(g, _req(p, script=[{"text": "a", "speaker": "x"}, {"text": "b", "speaker": "y"}])):
        raise ConformanceFailure(f"{mid}: a multi-speaker script was accepted without the capability")
    # ---- output invariants + progress ----
    events = []
    out = g.generate(_req(p), events.append)
    t = out.audio
    if t is None or out.images or out.video_frames:
        raise ConformanceFailure(f"{mid}: an audio generator must return exactly one audio track")
    if t.sample_rate not in caps.audio_sample_rates or t.channels < 1 or not t.samples or len(t.samples) % t.channels:
        raise ConformanceFailure(f"{mid}: bad track header ({t.sample_rate} Hz, {t.channels} ch, {len(t.samples)} samples)")
    if not all(math.isfinite(x) for x in t.samples):
        raise ConformanceFailure(f"{mid}: non-finite samples")
    secs = len(t.samples) / t.channels / t.sample_rate
    if caps.max_audio_duration_secs is not None and secs > 4 * caps.max_audio_duration_secs:
        raise ConformanceFailure(f"{mid}: {secs:.1f}s of audio for a short script")
    steps = [(e.current, e.total) for e in events if isinstance(e, ProgressStep)]
    if not steps or any(tt != steps[0][1] for _, tt in steps) or [c for c, _ in steps] != list(range(1, steps[0][1] + 1)):
        raise ConformanceFailure(f"{mid}: progress must count 1..=total with a fixed total; got {steps}")
    # ---- determinism ----
    again = g.generate(_req(p)).audio
    if again.samples != t.samples:
        raise ConformanceFailure(f"{mid}: the same seed produced different audio")
    # ---- cancellation ----
    pre = _req(p)
    pre.cancel = CancelFlag()
    pre.cancel.cancel()
    try:
        g.generate(pre)
    except Canceled:
        pass
    else:
        raise ConformanceFailure(f"{mid}: a pre-cancelled request must raise Canceled")
    mid_req = _req(p)

    def cancel_on_first(e):
        if isinstance(e, ProgressStep):
            mid_req.cancel.cancel()
    try:
        g.generate(mid_req, cancel_on_first)
    except Canceled:
        pass
    else:
        raise ConformanceFailure(f"{mid}: cancelling at the first step must raise Canceled")
    # ---- target duration ----
    if p.target_duration is not None:
        got = g.generate(_req(p, target_duration=p.target_duration)).audio
        gs = len(got.samples) / got.channels / got.sample_rate
        if abs(gs - p.target_duration) > p.duration_tolerance * p.target_duration and abs(gs - secs) < 1e-9:
            raise ConformanceFailure(f"{mid}: target_duration {p.target_duration}s had no effect ({gs:.2f}s both times)")
