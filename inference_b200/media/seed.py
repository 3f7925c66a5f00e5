"""Seed conventions shared by every media provider (parity: candle-gen/src/seed.rs:47-101).

* image `index` of a `count`-image request renders at `base_seed + index` (wrapping at 2**64), so the n-th image of
  a batch reproduces alone as a `count=1` request at that seed;
* per-step ancestral noise is keyed by `seed + STEP_RNG_SALT` so it never re-derives the prior noise;
* prior noise is drawn on the CPU from a seeded generator and then moved to the device, so the sample sequence does
  not depend on the GPU, the launch configuration or the number of ranks.
The draw uses torch's CPU Philox/MT stream, not the reference's Rust StdRng: seeds are reproducible within this
framework, not bit-compatible across the two."""
from __future__ import annotations

import time
from typing import Callable, TypeVar

import torch

T = TypeVar("T")
U64 = (1 << 64) - 1
STEP_RNG_SALT = 0x9E3779B97F4A7C15


def image_seed(base_seed: int, index: int) -> int:
    return (base_seed + index) & U64


def default_seed() -> int:
    """Non-deterministic: resolve it exactly once per generation and pass the result down."""
    return time.time_ns() & U64


def _generator(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed & 0x7FFFFFFFFFFFFFFF)


def seeded_normal(seed: int, n: int) -> torch.Tensor:
    return torch.randn(n, generator=_generator(seed), dtype=torch.float32)


def seeded_noise_nchw(seed: int, c: int, h: int, w: int, device="cpu") -> torch.Tensor:
    return seeded_normal(seed, c * h * w).view(1, c, h, w).to(device)


def for_each_image_seed(base_seed: int, count: int, body: Callable[[int], T]) -> list[T]:
    return [body(image_seed(base_seed, i)) for i in range(count)]
