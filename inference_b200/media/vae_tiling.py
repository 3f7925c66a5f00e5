"""Tiled VAE decode driver (candle-gen/src/vae_tiling.rs:53-330).

`decode_tiled` decodes overlapping latent tiles with any decoder callable and blends them with the plan's
trapezoidal masks into fp32 accumulators (sum of weighted tiles / sum of weights), so a constant field is
reconstructed exactly and seams cancel. The budget helpers pick the memory figure the planner works against:
an environment override, else a fraction of the device's total (or currently free) memory."""
from __future__ import annotations

import os
from typing import Callable

import torch

from ..contracts.errors import BackendError as GenError
from ..contracts.gen_core import video_tiling as vt
from . import gpu_probe


def decode_tiled(vae: vt.VaeTilingSpec, label: str, latent: torch.Tensor, cfg: vt.VideoTilingConfig,
                 decode_fn: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    """latent [B, C, F, H, W] -> decode_fn output [B, 3, F', H', W'], tiled when `cfg` says the extent needs it."""
    _, _, f, h, w = latent.shape
    if not cfg.needs_tiling(vae, f, h, w):
        return decode_fn(latent)
    return blend_plan(label, latent, cfg.plan(vae, f, h, w), decode_fn)


def blend_plan(label: str, latent: torch.Tensor, plan: vt.VideoTilePlan,
               decode_fn: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    dev = latent.device
    out = weights = None
    for t in plan.t:
        for hh in plan.h:
            for ww in plan.w:
                dec = decode_fn(latent[:, :, t.start:t.end, hh.start:hh.end, ww.start:ww.end])
                td, hd, wd = dec.shape[2:]
                at, ah, aw = (min(td, t.out_stop - t.out_start), min(hd, hh.out_stop - hh.out_start),
                              min(wd, ww.out_stop - ww.out_start))
                tm = torch.tensor(t.mask[:at], dtype=torch.float32, device=dev).view(1, 1, at, 1, 1)
                hm = torch.tensor(hh.mask[:ah], dtype=torch.float32, device=dev).view(1, 1, 1, ah, 1)
                wm = torch.tensor(ww.mask[:aw], dtype=torch.float32, device=dev).view(1, 1, 1, 1, aw)
                blend = tm * hm * wm
                if out is None:
                    b, c = dec.shape[:2]
                    out = torch.zeros((b, c, plan.out_f, plan.out_h, plan.out_w), dtype=torch.float32, device=dev)
                    weights = torch.zeros((1, 1, plan.out_f, plan.out_h, plan.out_w), dtype=torch.float32, device=dev)
                sl = (slice(None), slice(None), slice(t.out_start, t.out_start + at),
                      slice(hh.out_start, hh.out_start + ah), slice(ww.out_start, ww.out_start + aw))
                out[sl] += dec[:, :, :at, :ah, :aw].float() * blend
                weights[sl] += blend
    if out is None:
        raise GenError(f"{label}: tile-decode plan had no tiles")
    return (out / weights.clamp(min=1e-8)).to(latent.dtype)


def _env_gib(env_var: str) -> float | None:
    raw = os.environ.get(env_var)
    if raw is None:
        return None
    try:
        v = float(raw.strip())
    except ValueError:
        return None
    return v if v > 0 else None


def safe_budget_gib(env_var: str, safe_frac: float, default_gib: float,
                    total_probe: Callable[[], float | None] = gpu_probe.nvidia_smi_min_total_gib) -> float:
    """Override from `env_var` (GiB) > safe_frac x smallest GPU's total memory > default."""
    v = _env_gib(env_var)
    if v is not None:
        return v
    total = total_probe()
    return total * safe_frac if total is not None else default_gib


def free_aware_budget_gib(free_gib: float, safe_frac: float) -> float:
    return max(free_gib, 0.0) * safe_frac


def free_aware_safe_budget_gib(env_var: str, safe_frac: float, default_gib: float,
                               free_probe: Callable[[], float | None] = gpu_probe.nvidia_smi_rendered_free_gib
                               ) -> float:
    """As safe_budget_gib, but against the memory that is free now on the GPU this process uses (weights that are
    already resident shrink the budget)."""
    v = _env_gib(env_var)
    if v is not None:
        return v
    free = free_probe()
    return free_aware_budget_gib(free, safe_frac) if free is not None else default_gib


def plan_tiling(label: str, vae: vt.VaeTilingSpec, height: int, width: int, out_frames: int, safe_gib: float,
                candidates: vt.TileCandidates, cost_fn: vt.PeakCost) -> vt.VideoTilingConfig | None:
    """budgeted_plan with the failure turned into a message a user can act on."""
    try:
        return vt.budgeted_plan(vae, height, width, out_frames, safe_gib, candidates, cost_fn)
    except vt.TilingBudgetError as e:
        if e.kind == "accumulators":
            raise GenError(f"{label}: assembling a {width}x{height}x{out_frames} video needs ~{e.projected_gib:.0f} GB "
                           f"just for the output buffers, over the ~{e.safe_gib:.0f} GB safe VRAM budget. Reduce the "
                           "resolution or frame count.") from e
        raise GenError(f"{label}: a {width}x{height}x{out_frames} video peaks at ~{e.projected_gib:.0f} GB even with "
                       f"the smallest tile, over the ~{e.safe_gib:.0f} GB safe VRAM budget. Reduce the resolution or "
                       "frame count.") from e
