"""VAE tiling plans and memory adaptation policy (gen-core/src/tiling.rs:71-587, mempolicy.rs:38-257).

A `TilePlan` covers an H x W (x T) latent with overlapping tiles; decoded tiles are blended with a trapezoidal
ramp across the overlap so seams cancel exactly. `budgeted_plan` shrinks tiles until the estimated activation
footprint fits a byte budget; `plan_memory_adaptation` walks the lever ladder (sequential offload -> VAE tiling
-> branch quantisation -> resolution) and returns the first combination that fits."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class TilingConfig:
    tile: int              # latent-space tile edge
    overlap: int           # latent-space overlap between neighbours
    temporal_tile: int = 0
    temporal_overlap: int = 0


VAE_TILING_PRESETS = {"flux": TilingConfig(64, 16), "ltx": TilingConfig(32, 8, 8, 2), "wan": TilingConfig(32, 8, 8, 2),
                      "wan22": TilingConfig(32, 8, 6, 2), "qwen_image": TilingConfig(64, 16)}


@dataclass(frozen=True)
class Tile:
    y0: int
    y1: int
    x0: int
    x1: int


@dataclass
class TilePlan:
    height: int
    width: int
    tiles: list[Tile] = field(default_factory=list)
    overlap: int = 0

    def is_single(self) -> bool:
        return len(self.tiles) == 1


def _starts(extent: int, tile: int, overlap: int) -> list[int]:
    if tile >= extent:
        return [0]
    stride = max(1, tile - overlap)
    out = list(range(0, extent - tile, stride))
    out.append(extent - tile)
    return out


def plan_tiles(height: int, width: int, cfg: TilingConfig) -> TilePlan:
    tiles = [Tile(y, min(y + cfg.tile, height), x, min(x + cfg.tile, width))
             for y in _starts(height, cfg.tile, cfg.overlap) for x in _starts(width, cfg.tile, cfg.overlap)]
    return TilePlan(height, width, tiles, cfg.overlap)


def trapezoidal_mask(length: int, ramp_lo: int, ramp_hi: int) -> list[float]:
    """1-D blend weights: linear ramp up over ramp_lo samples, flat 1, ramp down over ramp_hi samples."""
    w = [1.0] * length
    for i in range(min(ramp_lo, length)):
        w[i] = (i + 1) / (ramp_lo + 1)
    for i in range(min(ramp_hi, length)):
        w[length - 1 - i] = min(w[length - 1 - i], (i + 1) / (ramp_hi + 1))
    return w


def budgeted_plan(height: int, width: int, cfg: TilingConfig, bytes_per_latent_pixel: int, budget_bytes: int
                  ) -> TilePlan:
    """Halve the tile edge (not below 2 x overlap + 8) until one tile's activations fit the budget."""
    tile = min(cfg.tile, max(height, width))
    floor_tile = 2 * cfg.overlap + 8
    while tile > floor_tile and tile * tile * bytes_per_latent_pixel > budget_bytes:
        tile = max(floor_tile, tile // 2)
    if height * width * bytes_per_latent_pixel <= budget_bytes:
        return TilePlan(height, width, [Tile(0, height, 0, width)], 0)
    return plan_tiles(height, width, TilingConfig(tile, cfg.overlap))


@dataclass
class MemoryPlan:
    sequential_offload: bool = False
    vae_tiling: bool = False
    quantize_branch: bool = False
    scale_resolution: float = 1.0
    fits: bool = True
    estimated_bytes: int = 0


def plan_memory_adaptation(budget_bytes: int, text_encoder_bytes: int, transformer_bytes: int, vae_bytes: int,
                           activation_bytes: int, vae_activation_bytes: int) -> MemoryPlan:
    """Lever ladder: Resident -> Sequential offload -> + VAE tiling -> + 4-bit branch -> lower resolution."""
    plan = MemoryPlan()

    def need(p: MemoryPlan) -> int:
        tr = transformer_bytes * (0.28 if p.quantize_branch else 1.0)
        act = activation_bytes * p.scale_resolution ** 2
        vact = (vae_activation_bytes / 8 if p.vae_tiling else vae_activation_bytes) * p.scale_resolution ** 2
        heavy = tr + vae_bytes + max(act, vact)
        return int(max(text_encoder_bytes, heavy) if p.sequential_offload else text_encoder_bytes + heavy)

    for lever in ("none", "sequential_offload", "vae_tiling", "quantize_branch"):
        if lever != "none":
            setattr(plan, lever, True)
        plan.estimated_bytes = need(plan)
        if plan.estimated_bytes <= budget_bytes:
            return plan
    for s in (0.75, 0.5, 0.375, 0.25):
        plan.scale_resolution = s
        plan.estimated_bytes = need(plan)
        if plan.estimated_bytes <= budget_bytes:
            return plan
    plan.fits = False
    return plan
