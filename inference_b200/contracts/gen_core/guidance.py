"""Classifier-free guidance family over LatentOps (gen-core/src/guidance.rs:40-299): plain CFG, CFG with std
rescale, adaptive projected guidance (APG, with momentum) and the CFG++ marker."""
from __future__ import annotations

import enum
import math


class GuidanceMethod(enum.Enum):
    CFG = "cfg"
    CFG_RESCALE = "cfg_rescale"
    APG = "apg"
    CFG_PP = "cfg_pp"

    @staticmethod
    def from_name(name: str) -> "GuidanceMethod | None":
        for m in GuidanceMethod:
            if m.value == name:
                return m
        return None


GUIDANCE_METHODS = tuple(m.value for m in GuidanceMethod)


def _flat(x):
    return x.reshape(-1).float() if hasattr(x, "reshape") else x


def _dot(a, b) -> float:
    if hasattr(a, "reshape"):
        return float((a.reshape(-1).float() * b.reshape(-1).float()).sum())
    return sum(u * v for u, v in zip(a, b))


def _std(x) -> float:
    if hasattr(x, "reshape"):
        return float(x.float().std(unbiased=False))
    n = len(x)
    m = sum(x) / n
    return math.sqrt(sum((v - m) ** 2 for v in x) / n)


def cfg(ops, cond, uncond, scale: float):
    """uncond + scale * (cond - uncond)."""
    return ops.axpy(1.0 - scale, uncond, scale, cond)


def cfg_rescale(ops, cond, uncond, scale: float, rescale: float = 0.7):
    """CFG followed by matching the guided std to the conditional std, blended by `rescale`."""
    g = cfg(ops, cond, uncond, scale)
    sg = _std(g)
    if sg <= 0.0:
        return g
    factor = _std(cond) / sg
    return ops.scale(g, rescale * factor + (1.0 - rescale))


class MomentumBuffer:
    def __init__(self, momentum: float):
        self.momentum = momentum
        self.running = None

    def update(self, ops, value):
        self.running = value if self.running is None else ops.axpy(1.0, value, self.momentum, self.running)
        return self.running


def apg_delta(ops, cond, uncond, eta: float = 0.0, norm_threshold: float = 0.0, momentum: MomentumBuffer | None = None):
    """The APG update direction: diff (optionally momentum-averaged and norm-clipped) split into components
    parallel and orthogonal to the conditional prediction; returns orthogonal + eta * parallel."""
    diff = ops.sub(cond, uncond)
    if momentum is not None:
        diff = momentum.update(ops, diff)
    if norm_threshold > 0.0:
        n = math.sqrt(max(_dot(diff, diff), 0.0))
        if n > norm_threshold:
            diff = ops.scale(diff, norm_threshold / n)
    cc = _dot(cond, cond)
    if cc <= 0.0:
        return diff
    coef = _dot(diff, cond) / cc
    parallel = ops.scale(cond, coef)
    orth = ops.sub(diff, parallel)
    return ops.axpy(1.0, orth, eta, parallel)


def apg(ops, cond, uncond, scale: float, eta: float = 0.0, norm_threshold: float = 0.0,
        momentum: MomentumBuffer | None = None):
    return ops.axpy(1.0, cond, scale - 1.0, apg_delta(ops, cond, uncond, eta, norm_threshold, momentum))
