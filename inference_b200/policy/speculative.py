"""Speculative-decoding policy: prompt-lookup n-gram proposer, greedy acceptance run, distribution-preserving
stochastic acceptance with residual resampling (core-llm/src/speculative.rs:32-156). RNG-free: uniform draws are
arguments, so the math is testable and the engine owns the random stream."""
from __future__ import annotations

import ctypes

from ._lib import f32_array, i32_array, lib


def ngram_propose(tokens: list[int], max_ngram: int, max_proposal: int) -> list[int]:
    out = (ctypes.c_int32 * max(1, max_proposal))()
    n = lib().swb_ngram_propose(i32_array(tokens), len(tokens), max_ngram, max_proposal, out)
    return list(out[:n])


def accept_greedy_run(target_argmax: list[int], drafts: list[int]) -> int:
    assert len(target_argmax) == len(drafts) + 1, "need a bonus slot past the drafts"
    return lib().swb_accept_greedy_run(i32_array(target_argmax), i32_array(drafts), len(drafts))


def sample_weighted(candidates: list[tuple[int, float]], u: float, fallback: int) -> int:
    ids = i32_array([c[0] for c in candidates])
    w = f32_array([c[1] for c in candidates])
    return lib().swb_sample_weighted(ids, w, len(candidates), u, fallback)


def accept_token(target: list[tuple[int, float]], draft: list[tuple[int, float]], proposed: int, u_accept: float,
                 u_resample: float) -> tuple[bool, int]:
    """Returns (accepted, token): the proposed token when accepted, else the residual resample."""
    tok = ctypes.c_int32()
    ok = lib().swb_accept_token(i32_array([t[0] for t in target]), f32_array([t[1] for t in target]), len(target),
                                i32_array([d[0] for d in draft]), f32_array([d[1] for d in draft]), len(draft),
                                proposed, u_accept, u_resample, ctypes.byref(tok))
    return bool(ok), tok.value
