"""Host token sampler (candle-llm/src/primitives/sampler.rs:19-256): SplitMix64 stream, constraint mask,
repetition penalty over a recent window, temperature, top-k, top-p nucleus (heap order: weight desc, index asc)
and an inverse-CDF categorical draw. Greedy and masked-greedy requests on a GPU go through the device argmax
kernel instead (see engine.decode)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from ._lib import F32P, I32P, U8P, i32_array, lib


class SplitMix64:
    INCREMENT = 0x9E3779B97F4A7C15

    def __init__(self, seed: int):
        self._s = ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def next_u64(self) -> int:
        return lib().swb_splitmix64_next(ctypes.byref(self._s))

    def next_f32(self) -> float:
        return lib().swb_splitmix64_next_f32(ctypes.byref(self._s))

    @property
    def state_ref(self):
        return ctypes.byref(self._s)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    repetition_context: int = 0

    def is_plain_greedy(self) -> bool:
        return self.temperature <= 0.0 and self.repetition_penalty == 1.0


def _prep(logits, allowed):
    v = np.ascontiguousarray(np.asarray(logits, dtype=np.float32).reshape(-1))
    a = None
    if allowed is not None:
        a = np.ascontiguousarray(np.asarray(allowed, dtype=np.uint8).reshape(-1))
    return v, a


def sample(logits, history: list[int], params: SamplingParams, rng: SplitMix64, allowed=None) -> int:
    v, a = _prep(logits, allowed)
    return lib().swb_sample(v.ctypes.data_as(F32P), v.size, i32_array(history), len(history), params.temperature,
                            params.top_p, params.top_k, params.repetition_penalty, params.repetition_context,
                            a.ctypes.data_as(U8P) if a is not None else None, a.size if a is not None else 0,
                            rng.state_ref)


def shaped_candidates(logits, history: list[int], params: SamplingParams, allowed=None) -> list[tuple[int, float]]:
    v, a = _prep(logits, allowed)
    ids = np.empty(v.size, dtype=np.int32)
    w = np.empty(v.size, dtype=np.float32)
    n = lib().swb_shaped_candidates(v.ctypes.data_as(F32P), v.size, i32_array(history), len(history),
                                    params.temperature, params.top_p, params.top_k, params.repetition_penalty,
                                    params.repetition_context, a.ctypes.data_as(U8P) if a is not None else None,
                                    a.size if a is not None else 0, ids.ctypes.data_as(I32P), w.ctypes.data_as(F32P),
                                    v.size)
    return [(int(ids[i]), float(w[i])) for i in range(n)]


def argmax_host(logits) -> int:
    v = np.asarray(logits, dtype=np.float32).reshape(-1)
    return int(np.argmax(v))  # first maximum: ties resolve to the lowest index
