"""Test tooling shared by media provider suites (candle-gen/src/testkit.rs:37-688): environment paths, PPM image IO,
image / vector similarity, and device-memory probes (allocator high-water marks and an nvidia-smi peak sampler)."""
from __future__ import annotations

import math
import os
import threading
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from ..contracts.gen_core.media import Image


def env_path(key: str) -> Path:
    """The directory a test needs, from the environment; a missing variable is a hard error naming the variable."""
    v = os.environ.get(key)
    if not v:
        raise RuntimeError(f"set {key} to run this test")
    return Path(v)


def env_path_opt(key: str) -> Path | None:
    v = os.environ.get(key)
    return Path(v) if v else None


def write_ppm(path: str | Path, img: Image) -> None:
    Path(path).write_bytes(img.to_ppm())


def read_ppm(path: str | Path) -> Image:
    """Binary P6 with maxval 255 (comments allowed in the header)."""
    data = Path(path).read_bytes()
    fields, pos = [], 0
    while len(fields) < 4:
        while pos < len(data) and data[pos:pos + 1].isspace():
            pos += 1
        if data[pos:pos + 1] == b"#":
            while pos < len(data) and data[pos:pos + 1] != b"\n":
                pos += 1
            continue
        end = pos
        while end < len(data) and not data[end:end + 1].isspace():
            end += 1
        fields.append(data[pos:end])
        pos = end
    if fields[0] != b"P6" or fields[3] != b"255":
        raise ValueError(f"{path}: not a binary 8-bit PPM")
    w, h = int(fields[1]), int(fields[2])
    return Image(w, h, data[pos + 1:pos + 1 + w * h * 3])


def mean_abs_diff(a: Image, b: Image) -> float:
    if (a.width, a.height) != (b.width, b.height):
        raise ValueError("image sizes differ")
    return sum(abs(x - y) for x, y in zip(a.pixels, b.pixels)) / max(1, len(a.pixels))


def cosine(a, b) -> float:
    dot = sum(x * y for x, y in zip(a, b))
    na, nb = math.sqrt(sum(x * x for x in a)), math.sqrt(sum(y * y for y in b))
    return dot / (na * nb) if na > 0 and nb > 0 else 0.0


def tensor_cosine(a, b) -> float:
    import torch

    x, y = a.detach().double().flatten(), b.detach().double().flatten()
    d = float(x.norm() * y.norm())
    return float(torch.dot(x, y)) / d if d > 0 else 0.0


def reset_cuda_mempool_high_water(ordinal: int = 0) -> bool:
    import torch

    if not torch.cuda.is_available():
        return False
    torch.cuda.reset_peak_memory_stats(ordinal)
    return True


def cuda_mempool_used_high_bytes(ordinal: int = 0) -> int | None:
    import torch

    return torch.cuda.max_memory_allocated(ordinal) if torch.cuda.is_available() else None


UsedProbe = Callable[[], "int | None"]        # MiB in use on the device right now


def used_mib(gpu: int = 0) -> int | None:
    from ..media.gpu_probe import _run

    out = _run(["--query-gpu=memory.used", "--format=csv,noheader,nounits", "-i", str(gpu)])
    try:
        return int(float(out.strip().splitlines()[0])) if out else None
    except (ValueError, IndexError):
        return None


class PeakSampler:
    """Polls device memory in a background thread and keeps the maximum (MiB)."""

    def __init__(self, probe: UsedProbe, interval_s: float = 0.05):
        self._probe, self._interval = probe, interval_s
        self._peak = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    @classmethod
    def start(cls, gpu: int = 0, interval_s: float = 0.05) -> "PeakSampler":
        return cls(lambda: used_mib(gpu), interval_s)

    def _loop(self) -> None:
        while not self._stop.is_set():
            v = self._probe()
            if v is not None and v > self._peak:
                self._peak = v
            self._stop.wait(self._interval)

    def stop(self) -> int:
        self._stop.set()
        self._thread.join(timeout=5)
        v = self._probe()
        if v is not None and v > self._peak:
            self._peak = v
        return self._peak


@dataclass
class VramReport:
    baseline_mib: int
    load_peak_mib: int
    gen_peak_mib: int

    @property
    def load_delta_gb(self) -> float:
        return max(0, self.load_peak_mib - self.baseline_mib) / 1024.0

    @property
    def gen_delta_gb(self) -> float:
        return max(0, self.gen_peak_mib - self.baseline_mib) / 1024.0

    def assert_trustworthy(self, max_baseline_gb: float) -> "VramReport":
        """A busy device before the run makes the deltas meaningless."""
        if self.baseline_mib / 1024.0 > max_baseline_gb:
            raise AssertionError(f"device was not idle: {self.baseline_mib / 1024.0:.1f} GB in use before the run")
        return self


class VramProbe:
    """Baseline, load-phase and generation-phase peaks of one provider run."""

    def __init__(self, probe: UsedProbe, interval_s: float = 0.05):
        self._probe, self._interval = probe, interval_s
        self.baseline_mib = probe() or 0
        self.load_peak_mib = self.gen_peak_mib = self.baseline_mib

    @classmethod
    def start(cls, gpu: int = 0) -> "VramProbe":
        return cls(lambda: used_mib(gpu))

    def assert_idle(self, max_baseline_gb: float) -> "VramProbe":
        if self.baseline_mib / 1024.0 > max_baseline_gb:
            raise AssertionError(f"device was not idle: {self.baseline_mib / 1024.0:.1f} GB in use")
        return self

    def phase(self) -> PeakSampler:
        return PeakSampler(self._probe, self._interval)

    def end_load(self, phase: PeakSampler) -> None:
        self.load_peak_mib = max(self.load_peak_mib, phase.stop())

    def end_gen(self, phase: PeakSampler) -> None:
        self.gen_peak_mib = max(self.gen_peak_mib, phase.stop())

    def report(self) -> VramReport:
        return VramReport(self.baseline_mib, self.load_peak_mib, self.gen_peak_mib)
