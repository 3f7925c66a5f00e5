"""Device memory probe through `nvidia-smi`, resolved from trusted absolute paths only
(candle-gen/src/gpu.rs:72-128): the binary is never looked up through PATH, so a writable PATH entry cannot
substitute another program. The probe only reads."""
from __future__ import annotations

import os
import subprocess
from pathlib import Path
from typing import Callable

_resolved: list[Path | None] = []


def candidate_paths() -> list[Path]:
    out = [Path("/usr/bin/nvidia-smi"), Path("/usr/local/bin/nvidia-smi")]
    cuda = os.environ.get("CUDA_PATH")
    if cuda:
        out.append(Path(cuda) / "bin" / "nvidia-smi")
    return out


def first_existing(candidates: list[Path]) -> Path | None:
    for p in candidates:
        if p.exists():
            return p
    return None


def resolve_nvidia_smi() -> Path | None:
    if not _resolved:
        _resolved.append(first_existing(candidate_paths()))
    return _resolved[0]


def parse_min_mib_line_gib(text: str) -> float | None:
    """Smallest positive MiB figure over the lines (one per GPU), in GiB; None when there is none."""
    vals = []
    for line in text.splitlines():
        try:
            v = float(line.strip())
        except ValueError:
            continue
        if v > 0:
            vals.append(v)
    return min(vals) / 1024.0 if vals else None


def parse_rendered_ordinal(raw: str | None) -> int | None:
    """The GPU this process renders on: first entry of CUDA_VISIBLE_DEVICES when it is a plain ordinal, 0 when the
    variable is unset, None for UUID / MIG forms (they cannot be passed to `-i` as an index)."""
    if raw is None:
        return 0
    first = raw.split(",")[0].strip()
    return int(first) if first.isdigit() else None


Runner = Callable[[list[str]], "str | None"]


def _run(args: list[str]) -> str | None:
    exe = resolve_nvidia_smi()
    if exe is None:
        return None
    try:
        r = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=20)
    except (OSError, subprocess.SubprocessError):
        return None
    return r.stdout if r.returncode == 0 else None


def _query_min_gib(field: str, run: Runner) -> float | None:
    out = run([f"--query-gpu={field}", "--format=csv,noheader,nounits"])
    return parse_min_mib_line_gib(out) if out is not None else None


def nvidia_smi_min_total_gib(run: Runner = _run) -> float | None:
    return _query_min_gib("memory.total", run)


def nvidia_smi_min_free_gib(run: Runner = _run) -> float | None:
    return _query_min_gib("memory.free", run)


def nvidia_smi_rendered_free_gib(run: Runner = _run, env: dict | None = None) -> float | None:
    """Free memory of the GPU this process uses; falls back to the minimum over all GPUs."""
    env = os.environ if env is None else env
    ordinal = parse_rendered_ordinal(env.get("CUDA_VISIBLE_DEVICES"))
    if ordinal is not None:
        out = run(["--query-gpu=memory.free", "--format=csv,noheader,nounits", "-i", str(ordinal)])
        got = parse_min_mib_line_gib(out) if out is not None else None
        if got is not None:
            return got
    return nvidia_smi_min_free_gib(run)
