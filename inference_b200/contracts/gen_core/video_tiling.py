"""Spatio-temporal VAE tiling policy for video and large-image decoders (gen-core/src/tiling.rs:65-660).

A `VaeTilingSpec` describes a decoder (spatial / temporal upscale, causal first frame, channel width at full
resolution); a `VideoTilingConfig` is tile and overlap sizes in OUTPUT pixels / frames; `plan()` turns a latent
extent into per-axis tiles carrying the output range each decodes to and the trapezoidal blend mask over that range.
`budgeted_plan` picks the largest tile whose projected peak memory fits a budget, and also tiles when a single pass
would write more than 2^31 - 1 elements in one full-resolution activation."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Callable, Sequence

MAX_WRITABLE_ELEMS = 2 ** 31 - 1


@dataclass(frozen=True)
class VaeTilingSpec:
    spatial_scale: int
    temporal_scale: int
    causal_temporal: bool
    full_res_channels: int

    def writable_frame_cap(self, out_h: int, out_w: int) -> int:
        per_frame = self.full_res_channels * out_h * out_w
        return (2 ** 63 - 1) if per_frame <= 0 else MAX_WRITABLE_ELEMS // per_frame

    def with_channels(self, c: int) -> "VaeTilingSpec":
        return replace(self, full_res_channels=c)


LTX = VaeTilingSpec(32, 8, True, 8)
WAN = VaeTilingSpec(8, 4, False, 96)
WAN22 = VaeTilingSpec(16, 4, True, 64)
QWEN_IMAGE = VaeTilingSpec(8, 1, False, 96)


@dataclass(frozen=True)
class SpatialTiling:
    tile_px: int
    overlap_px: int


@dataclass(frozen=True)
class TemporalTiling:
    tile_frames: int
    overlap_frames: int


@dataclass(frozen=True)
class AxisTile:
    start: int           # latent range [start, end)
    end: int
    out_start: int       # output range this tile is blended into
    out_stop: int
    mask: tuple[float, ...]


@dataclass(frozen=True)
class VideoTilePlan:
    t: tuple[AxisTile, ...]
    h: tuple[AxisTile, ...]
    w: tuple[AxisTile, ...]
    out_f: int
    out_h: int
    out_w: int


def _f32(x: float) -> float:
    import struct

    return struct.unpack("f", struct.pack("f", x))[0]


def trapezoidal_mask(length: int, ramp_left: int, ramp_right: int, left_from_0: bool) -> list[float]:
    """Blend weights along one axis: a fade-in over ramp_left samples (starting at exactly 0 when left_from_0, else
    strictly inside (0, 1)), ones, then a fade-out over ramp_right samples that never reaches 0."""
    length = max(1, length)
    ramp_left = min(max(ramp_left, 0), length)
    ramp_right = min(max(ramp_right, 0), length)
    mask = [1.0] * length
    if ramp_left > 0:
        interval = ramp_left + 1 if left_from_0 else ramp_left + 2
        full = [_f32(i / (interval - 1.0)) for i in range(interval)]
        fade = full[: interval - 1] if left_from_0 else full[1: interval - 1]
        for i in range(min(ramp_left, len(fade))):
            mask[i] = _f32(mask[i] * fade[i])
    if ramp_right > 0:
        for i in range(ramp_right):
            v = _f32((ramp_right + 1.0 - (i + 1.0)) / (ramp_right + 1.0))
            j = length - ramp_right + i
            mask[j] = _f32(mask[j] * v)
    return [min(1.0, max(0.0, v)) for v in mask]


def split_spatial(size: int, overlap: int, dim: int):
    size = max(1, size)
    overlap = min(max(overlap, 0), size - 1)
    if dim <= size:
        return [0], [dim], [0], [0]
    amount = (dim + size - 2 * overlap - 1) // (size - overlap)
    starts = [i * (size - overlap) for i in range(amount)]
    ends = [s + size for s in starts]
    ends[-1] = dim
    left = [overlap] * amount
    left[0] = 0
    right = [overlap] * amount
    right[-1] = 0
    return starts, ends, left, right


def split_temporal(size: int, overlap: int, dim: int):
    """A causal decoder emits 1 + (n - 1) * scale frames, so every tile but the first starts one latent frame early
    and blends over one more."""
    starts, ends, left, right = split_spatial(size, overlap, dim)
    for i in range(1, len(starts)):
        starts[i] -= 1
        left[i] += 1
    return starts, ends, left, right


def _spatial_tiles(tile: int, overlap: int, dim: int, scale: int) -> tuple[AxisTile, ...]:
    starts, ends, left, right = split_spatial(tile, overlap, dim)
    out = []
    for i, b in enumerate(starts):
        o0, o1 = b * scale, ends[i] * scale
        out.append(AxisTile(b, ends[i], o0, o1, tuple(trapezoidal_mask(o1 - o0, left[i] * scale, right[i] * scale,
                                                                       False))))
    return tuple(out)


def _temporal_tiles(tile: int, overlap: int, dim: int, scale: int, causal: bool) -> tuple[AxisTile, ...]:
    if not causal:
        return _spatial_tiles(tile, overlap, dim, scale)
    starts, ends, left, right = split_temporal(tile, overlap, dim)
    out = []
    for i, b in enumerate(starts):
        o0, o1 = b * scale, 1 + (ends[i] - 1) * scale
        ls = 1 + (left[i] - 1) * scale if left[i] > 0 else 0
        out.append(AxisTile(b, ends[i], o0, o1, tuple(trapezoidal_mask(o1 - o0, ls, right[i] * scale, True))))
    return tuple(out)


@dataclass(frozen=True)
class VideoTilingConfig:
    spatial: SpatialTiling | None = None
    temporal: TemporalTiling | None = None

    @classmethod
    def default_preset(cls):
        return cls(SpatialTiling(512, 64), TemporalTiling(64, 24))

    @classmethod
    def aggressive(cls):
        return cls(SpatialTiling(256, 64), TemporalTiling(32, 8))

    @classmethod
    def conservative(cls):
        return cls(SpatialTiling(768, 64), TemporalTiling(96, 24))

    @classmethod
    def spatial_only(cls, tile_px: int, overlap_px: int):
        return cls(SpatialTiling(tile_px, overlap_px), None)

    @classmethod
    def temporal_only(cls, tile_frames: int, overlap_frames: int):
        return cls(None, TemporalTiling(tile_frames, overlap_frames))

    @classmethod
    def auto(cls, height: int, width: int, num_frames: int) -> "VideoTilingConfig | None":
        needs_s, needs_t = height > 512 or width > 512, num_frames > 65
        if not needs_s and not needs_t:
            return None
        est_gb = 3.0 * num_frames * height * width * 4.0 / 2 ** 30
        if est_gb > 2.0 or (height * width > 768 * 1024 and num_frames > 100):
            return cls.aggressive()
        spatial = SpatialTiling(384 if max(height, width) > 1024 else 512, 64) if needs_s else None
        temporal = None
        if needs_t:
            temporal = TemporalTiling(*((32, 8) if num_frames > 200 else (48, 16) if num_frames > 100 else (64, 24)))
        return cls(spatial, temporal)

    def needs_tiling(self, vae: VaeTilingSpec, f: int, h: int, w: int) -> bool:
        s = self.spatial is not None and (h > self.spatial.tile_px // vae.spatial_scale
                                          or w > self.spatial.tile_px // vae.spatial_scale)
        t = self.temporal is not None and f > self.temporal.tile_frames // vae.temporal_scale
        return s or t

    def plan(self, vae: VaeTilingSpec, f: int, h: int, w: int) -> VideoTilePlan:
        if self.temporal is not None:
            t_tile, t_over = (self.temporal.tile_frames // vae.temporal_scale,
                              self.temporal.overlap_frames // vae.temporal_scale)
        else:
            t_tile, t_over = f, 0
        if self.spatial is not None:
            s_tile, s_over = self.spatial.tile_px // vae.spatial_scale, self.spatial.overlap_px // vae.spatial_scale
        else:
            s_tile, s_over = max(h, w), 0
        return VideoTilePlan(
            t=_temporal_tiles(t_tile, t_over, f, vae.temporal_scale, vae.causal_temporal),
            h=_spatial_tiles(s_tile, s_over, h, vae.spatial_scale),
            w=_spatial_tiles(s_tile, s_over, w, vae.spatial_scale),
            out_f=1 + (f - 1) * vae.temporal_scale if vae.causal_temporal else f * vae.temporal_scale,
            out_h=h * vae.spatial_scale, out_w=w * vae.spatial_scale)


@dataclass(frozen=True)
class TileCandidates:
    spatial_px: Sequence[int]
    spatial_overlap_px: int
    temporal: Sequence[tuple[int, int]]       # (tile_frames, overlap_frames)


class TilingBudgetError(Exception):
    def __init__(self, kind: str, projected_gib: float, safe_gib: float):
        self.kind, self.projected_gib, self.safe_gib = kind, projected_gib, safe_gib
        what = ("the output buffers alone need" if kind == "accumulators" else "peaks at")
        tail = "" if kind == "accumulators" else " even with the smallest tile"
        super().__init__(f"video VAE decode: {what} ~{projected_gib:.0f} GB{tail}, over the ~{safe_gib:.0f} GB safe "
                         "budget; reduce the resolution or frame count")


PeakCost = Callable[[int, int, int, int, int, int], float]   # (out_f, out_h, out_w, tile_f, tile_h, tile_w) -> GiB


def budgeted_plan(vae: VaeTilingSpec, out_height: int, out_width: int, out_frames: int, safe_gib: float,
                  candidates: TileCandidates, peak_cost: PeakCost) -> VideoTilingConfig | None:
    """None when a single pass fits (memory and the 2^31-1 element write bound); else the candidate with the most
    voxels per tile whose projected peak fits. Raises TilingBudgetError when nothing can fit."""
    h, w, f = out_height, out_width, out_frames
    frame_cap = vae.writable_frame_cap(h, w)
    if frame_cap == 0:
        raise TilingBudgetError("accumulators", peak_cost(f, h, w, 0, 0, 0), safe_gib)
    single = peak_cost(f, h, w, f, h, w)
    if single <= safe_gib and f <= frame_cap:
        return None
    accum = peak_cost(f, h, w, 0, 0, 0)
    if accum >= safe_gib:
        raise TilingBudgetError("accumulators", accum, safe_gib)
    max_sp = max(h, w)
    spatial = [s for s in candidates.spatial_px if s < max_sp] + [max_sp]
    temporal = [(t, o) for t, o in candidates.temporal if t < f] + [(f, 0)]
    best = None
    min_peak = single
    for s in spatial:
        th, tw = min(s, h), min(s, w)
        for t, t_over in temporal:
            tf = min(t, f)
            if th == h and tw == w and tf == f:
                continue
            if vae.full_res_channels * tf * th * tw > MAX_WRITABLE_ELEMS:
                continue
            peak = peak_cost(f, h, w, tf, th, tw)
            min_peak = min(min_peak, peak)
            if peak > safe_gib:
                continue
            vox = tf * th * tw
            if best is None or vox > best[0]:
                best = (vox, s, t, t_over)
    if best is None:
        raise TilingBudgetError("smallest_tile", min_peak, safe_gib)
    _, s, t, t_over = best
    return VideoTilingConfig(SpatialTiling(s, candidates.spatial_overlap_px) if s < max_sp else None,
                             TemporalTiling(t, t_over) if t < f else None)
