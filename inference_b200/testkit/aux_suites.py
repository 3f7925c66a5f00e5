"""Conformance suites for the non-generator provider kinds (gen-core-testkit/src/{transcriber,voice_embedder,
captioner,audio_embedder,trainer}.rs): the guarantees the traits promise but cannot type. Each check raises
`ConformanceFailure` with the broken law in its message; `*_conformance` runs a provider kind's full list."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable

from ..contracts.errors import Canceled
from ..contracts.gen_core.media import AudioTrack, Image
from ..contracts.gen_core.traits import TrainingConfig
from .generator import ConformanceFailure


def _finite(v) -> bool:
    return all(isinstance(x, (int, float)) and math.isfinite(x) for x in v)


def _tone(seconds: float, rate: int = 16_000, hz: float = 220.0, amp: float = 0.1) -> AudioTrack:
    n = int(seconds * rate)
    return AudioTrack(rate, 1, [amp * math.sin(2 * math.pi * hz * i / rate) for i in range(n)])


# ---- transcriber ---------------------------------------------------------------------------------------------------------
@dataclass
class TranscriberProfile:
    audio: AudioTrack = field(default_factory=lambda: _tone(1.0))
    language: str | None = "en"


def check_transcriber_output(t, p: TranscriberProfile) -> None:
    segs = t.transcribe(p.audio, p.language)
    if not isinstance(segs, list):
        raise ConformanceFailure("transcribe must return a list of segments")
    last = 0.0
    for s in segs:
        if not (math.isfinite(s.start) and math.isfinite(s.end)) or s.start < 0 or s.end < s.start:
            raise ConformanceFailure(f"segment times must be finite and ordered, got [{s.start}, {s.end}]")
        if s.start + 1e-6 < last:
            raise ConformanceFailure("segments must be in time order")
        last = s.start
        if not isinstance(s.text, str) or not s.text.strip():
            raise ConformanceFailure("a segment must carry non-empty text")
    again = t.transcribe(p.audio, p.language)
    if [(s.start, s.end, s.text) for s in segs] != [(s.start, s.end, s.text) for s in again]:
        raise ConformanceFailure("greedy transcription must be deterministic")


def check_transcriber_rejects_empty(t, p: TranscriberProfile) -> None:
    try:
        t.transcribe(AudioTrack(p.audio.sample_rate, 1, []), p.language)
    except Exception:
        return
    raise ConformanceFailure("empty audio must be a typed error, not an empty transcript")


def transcriber_conformance(t, p: TranscriberProfile | None = None) -> None:
    p = p or TranscriberProfile()
    d = t.descriptor()
    if not d.id or not d.backend:
        raise ConformanceFailure("descriptor must name an id and a backend")
    check_transcriber_output(t, p)
    check_transcriber_rejects_empty(t, p)


# ---- voice / audio / image / text embedders ------------------------------------------------------------------------------
def voice_embedder_conformance(e, clip: AudioTrack | None = None) -> None:
    clip = clip or _tone(1.5)
    v = e.embed(clip)
    dim = e.descriptor().extra.get("dim")
    if not v or not _finite(v):
        raise ConformanceFailure("the embedding must be non-empty and finite")
    if dim is not None and len(v) != dim:
        raise ConformanceFailure(f"embedding length {len(v)} differs from the advertised dim {dim}")
    if e.embed(clip) != v:
        raise ConformanceFailure("embedding the same clip twice must give the same vector")
    try:
        e.embed(AudioTrack(clip.sample_rate, 1, []))
    except Exception:
        return
    raise ConformanceFailure("a degenerate (empty) clip must be rejected with an error")


def vector_embedder_conformance(e, inputs: list, unit_norm: bool = True) -> None:
    """Image / text / audio embedders: one finite vector per input, equal lengths, deterministic, optionally unit norm."""
    out = e.embed(inputs)
    if len(out) != len(inputs):
        raise ConformanceFailure(f"{len(inputs)} inputs produced {len(out)} vectors")
    dims = {len(v) for v in out}
    if len(dims) != 1 or 0 in dims or not all(_finite(v) for v in out):
        raise ConformanceFailure("vectors must be finite and of one common length")
    if unit_norm and any(abs(math.sqrt(sum(x * x for x in v)) - 1) > 1e-3 for v in out):
        raise ConformanceFailure("vectors must be L2-normalised")
    if e.embed(inputs) != out:
        raise ConformanceFailure("embedding must be deterministic")
    if e.embed([]) != []:
        raise ConformanceFailure("no inputs must give no vectors")


# ---- captioner -----------------------------------------------------------------------------------------------------------
def captioner_conformance(c, image: Image | None = None, prompt: str | None = None, budget: int = 4,
                          count_tokens: Callable[[str], int] | None = None) -> None:
    image = image or Image(32, 32, bytes([127]) * (32 * 32 * 3))
    a = c.caption(image, prompt, budget)
    if not isinstance(a, str):
        raise ConformanceFailure("caption must return text")
    if count_tokens is not None and count_tokens(a) > budget:
        raise ConformanceFailure(f"caption exceeds max_new_tokens={budget}")
    if c.caption(image, prompt, budget) != a:
        raise ConformanceFailure("greedy captioning must be deterministic")
    if c.caption(image, prompt, 0).strip():
        raise ConformanceFailure("a zero token budget must give an empty caption")


# ---- trainer -------------------------------------------------------------------------------------------------------------
@dataclass
class TrainerProfile:
    dataset_dir: Path
    output_dir: Path
    steps: int = 3
    rank: int = 2


def _cfg(p: TrainerProfile, **kw) -> TrainingConfig:
    base = dict(dataset_dir=p.dataset_dir, output_dir=p.output_dir, steps=p.steps, rank=p.rank, alpha=float(p.rank))
    base.update(kw)
    return TrainingConfig(**base)


def check_trainer_validate(t, p: TrainerProfile) -> None:
    t.validate(_cfg(p))
    for bad, why in ((dict(steps=0), "zero steps"), (dict(rank=0), "zero rank"), (dict(learning_rate=-1.0), "negative lr"),
                     (dict(dataset_dir=p.dataset_dir / "missing"), "a missing dataset")):
        try:
            t.validate(_cfg(p, **bad))
        except Exception:
            continue
        raise ConformanceFailure(f"validate must reject {why}")


def check_trainer_progress(t, p: TrainerProfile) -> Path:
    seen = []
    out = t.train(_cfg(p), seen.append)
    steps = [e.step for e in seen]
    if steps != sorted(steps) or not steps or steps[-1] != p.steps or any(e.total != p.steps for e in seen):
        raise ConformanceFailure(f"progress must count up to total={p.steps}, got {steps}")
    if not Path(out).is_file() or Path(out).stat().st_size == 0:
        raise ConformanceFailure("train must return the adapter file it wrote")
    return Path(out)


def check_trainer_cancellation(t, p: TrainerProfile) -> None:
    cfg = _cfg(p, steps=max(4, p.steps))

    def on(e):
        if e.step >= 1:
            cfg.cancel.cancel()
    try:
        t.train(cfg, on)
    except Canceled:
        return
    raise ConformanceFailure("a cancel raised during training must end it with the typed Canceled error")


def trainer_conformance(t, p: TrainerProfile) -> None:
    check_trainer_validate(t, p)
    check_trainer_progress(t, p)
    check_trainer_cancellation(t, p)
