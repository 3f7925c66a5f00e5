"""The five latent operations every sampler is written against (gen-core/src/sampling/latent_ops.rs:26-63):
scale, add, sub, axpy (a*x + b*y) and seeded randn_like. `CpuLatentOps` works on plain float lists (the
tensor-free reference the unit tests use); `TorchLatentOps` works on torch tensors on any device and draws noise
from a CPU generator keyed by (seed, step) so results do not depend on the launch configuration."""
from __future__ import annotations

import abc
import random

import torch


class LatentOps(abc.ABC):
    @abc.abstractmethod
    def scale(self, x, s: float): ...
    @abc.abstractmethod
    def add(self, x, y): ...
    @abc.abstractmethod
    def sub(self, x, y): ...
    @abc.abstractmethod
    def axpy(self, a: float, x, b: float, y): ...
    @abc.abstractmethod
    def randn_like(self, x, seed: int, step: int): ...


class CpuLatentOps(LatentOps):
    def scale(self, x, s):
        return [v * s for v in x]

    def add(self, x, y):
        return [a + b for a, b in zip(x, y)]

    def sub(self, x, y):
        return [a - b for a, b in zip(x, y)]

    def axpy(self, a, x, b, y):
        return [a * u + b * v for u, v in zip(x, y)]

    def randn_like(self, x, seed, step):
        rng = random.Random((seed * 0x9E3779B97F4A7C15 + step) & 0xFFFFFFFFFFFFFFFF)
        return [rng.gauss(0.0, 1.0) for _ in x]


STEP_RNG_SALT = 0x5DEECE66D


class TorchLatentOps(LatentOps):
    def scale(self, x, s):
        return x * s

    def add(self, x, y):
        return x + y

    def sub(self, x, y):
        return x - y

    def axpy(self, a, x, b, y):
        if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and y.is_contiguous():
            from ....ops.dit import axpy as fused_axpy

            return fused_axpy(a, x, b, y)
        return a * x + b * y

    def randn_like(self, x, seed, step):
        g = torch.Generator().manual_seed((seed ^ (STEP_RNG_SALT * (step + 1))) & 0x7FFFFFFFFFFFFFFF)
        return torch.randn(x.shape, generator=g, dtype=torch.float32).to(device=x.device, dtype=x.dtype)
