"""Memory adaptation policy (gen-core/src/mempolicy.rs:38-257): which levers a lane engages, in cost order, to fit
a generation under a memory budget - sequential text-encoder residency, tiled VAE decode, a quantised control branch,
and only then a lower resolution. Pure arithmetic over projected stage peaks; no device access."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, Sequence

from .runtime import OffloadPolicy


class Lever(enum.IntEnum):
    SEQUENTIAL_RESIDENCY = 0
    VAE_DECODE_TILING = 1
    BRANCH_QUANT = 2
    RESOLUTION_REDUCTION = 3


@dataclass(frozen=True)
class StagePeaks:
    """Projected peaks (GiB) of the two heavy stages, text encoder excluded."""
    denoise_ex_text_gib: float
    decode_ex_text_gib: float
    decode_tiled_floor_ex_text_gib: float | None = None      # None: this lane's decoder cannot tile


@dataclass(frozen=True)
class LaneLevers:
    text_resident_gib: float
    supports_sequential: bool
    branch_quant_saves_gib: float
    resolution_scales: Sequence[float] = ()                  # descending, each < 1

    def residency_available(self) -> bool:
        return self.supports_sequential and self.text_resident_gib > 0.0


@dataclass
class AdaptationPlan:
    residency: OffloadPolicy = OffloadPolicy.RESIDENT
    tile_decode: bool = False
    quantize_branch: bool = False
    resolution_scale: float = 1.0
    projected_peak_gib: float = 0.0
    engaged: list[Lever] = field(default_factory=list)
    feasible: bool = True


def _engage(peaks: StagePeaks, levers: LaneLevers, safe: float) -> tuple[float, float, list[Lever]]:
    text = levers.text_resident_gib
    engaged: list[Lever] = []
    sequential = False
    denoise, decode = peaks.denoise_ex_text_gib + text, peaks.decode_ex_text_gib + text
    if (denoise > safe or decode > safe) and levers.residency_available():
        sequential = True
        denoise, decode = peaks.denoise_ex_text_gib, peaks.decode_ex_text_gib
        engaged.append(Lever.SEQUENTIAL_RESIDENCY)
    resident_text = 0.0 if sequential else text
    if decode > safe and peaks.decode_tiled_floor_ex_text_gib is not None:
        decode = peaks.decode_tiled_floor_ex_text_gib + resident_text
        engaged.append(Lever.VAE_DECODE_TILING)
    if (denoise > safe or decode > safe) and levers.branch_quant_saves_gib > 0.0:
        denoise = max(denoise - levers.branch_quant_saves_gib, 0.0)
        decode = max(decode - levers.branch_quant_saves_gib, 0.0)
        engaged.append(Lever.BRANCH_QUANT)
    return denoise, decode, engaged


def _plan(attempt, scale: float, feasible: bool) -> AdaptationPlan:
    denoise, decode, engaged = attempt
    engaged = list(engaged)
    plan = AdaptationPlan(
        residency=OffloadPolicy.SEQUENTIAL if Lever.SEQUENTIAL_RESIDENCY in engaged else OffloadPolicy.RESIDENT,
        tile_decode=Lever.VAE_DECODE_TILING in engaged, quantize_branch=Lever.BRANCH_QUANT in engaged,
        resolution_scale=scale, projected_peak_gib=max(denoise, decode), feasible=feasible)
    if scale < 1.0:
        engaged.append(Lever.RESOLUTION_REDUCTION)
    plan.engaged = engaged
    return plan


def plan_memory_adaptation(safe_gib: float, levers: LaneLevers, peaks_at: Callable[[float], StagePeaks]
                           ) -> AdaptationPlan:
    """The cheapest lever set that fits `safe_gib`: nothing when the resident plan fits; else the levers in cost order
    at full resolution; else the largest resolution scale at which they suffice; else the last attempt, marked
    infeasible, with its projected peak."""
    full = peaks_at(1.0)
    text = levers.text_resident_gib
    rd, rc = full.denoise_ex_text_gib + text, full.decode_ex_text_gib + text
    if rd <= safe_gib and rc <= safe_gib:
        return AdaptationPlan(projected_peak_gib=max(rd, rc))
    fits = lambda a: a[0] <= safe_gib and a[1] <= safe_gib
    attempt = _engage(full, levers, safe_gib)
    if fits(attempt):
        return _plan(attempt, 1.0, True)
    last, last_scale = attempt, 1.0
    for scale in levers.resolution_scales:
        attempt = _engage(peaks_at(scale), levers, safe_gib)
        if fits(attempt):
            return _plan(attempt, scale, True)
        last, last_scale = attempt, scale
    return _plan(last, last_scale, False)
