"""ctypes signatures of the host policy library (libswb200_host.so)."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_int32, c_long, c_uint8, c_uint64, c_void_p

from .._native import host

_DECLARED = False
I32P, F32P, U8P, U64P, LP = POINTER(c_int32), POINTER(c_float), POINTER(c_uint8), POINTER(c_uint64), POINTER(c_long)


def lib() -> ctypes.CDLL:
    global _DECLARED
    L = host()
    if _DECLARED:
        return L

    def sig(name, args, res=c_int):
        f = getattr(L, name)
        f.argtypes, f.restype = args, res

    sig("swb_alloc_new", [c_long], c_void_p)
    sig("swb_alloc_free", [c_void_p], None)
    for n in ("alloc", "live", "peak", "shared", "capacity"):
        sig(f"swb_alloc_{n}", [c_void_p], c_long)
    sig("swb_alloc_retain", [c_void_p, c_long])
    sig("swb_alloc_release", [c_void_p, c_long])
    sig("swb_alloc_refcount", [c_void_p, c_long])
    sig("swb_sched_new", [], c_void_p)
    sig("swb_sched_free", [c_void_p], None)
    sig("swb_sched_admit", [c_void_p, c_long, c_long, I32P, c_long], c_long)
    sig("swb_sched_len", [c_void_p], c_long)
    sig("swb_sched_record", [c_void_p, c_long, c_int32])
    sig("swb_sched_finish_reason", [c_void_p, c_long])
    sig("swb_sched_generated", [c_void_p, c_long, I32P, c_long], c_long)
    sig("swb_sched_prompt_len", [c_void_p, c_long], c_long)
    sig("swb_sched_offset", [c_void_p, c_long], c_long)
    sig("swb_sched_list", [c_void_p, c_int, LP, c_long], c_long)
    sig("swb_prefix_new", [c_long], c_void_p)
    sig("swb_prefix_free", [c_void_p], None)
    sig("swb_prefix_len", [c_void_p], c_long)
    sig("swb_prefix_contains", [c_void_p, c_uint64])
    sig("swb_prefix_longest_match", [c_void_p, I32P, c_long, U64P, LP])
    sig("swb_prefix_insert", [c_void_p, I32P, c_long, U64P, U64P, c_long], c_long)
    sig("swb_ngram_propose", [I32P, c_long, c_long, c_long, I32P], c_long)
    sig("swb_accept_greedy_run", [I32P, I32P, c_long], c_long)
    sig("swb_sample_weighted", [I32P, F32P, c_long, c_float, c_int32], c_int32)
    sig("swb_accept_token", [I32P, F32P, c_long, I32P, F32P, c_long, c_int32, c_float, c_float, I32P])
    sig("swb_splitmix64_next", [U64P], c_uint64)
    sig("swb_splitmix64_next_f32", [U64P], c_float)
    sig("swb_sample", [F32P, c_long, I32P, c_long, c_float, c_float, c_long, c_float, c_long, U8P, c_long, U64P],
        c_int32)
    sig("swb_shaped_candidates", [F32P, c_long, I32P, c_long, c_float, c_float, c_long, c_float, c_long, U8P, c_long,
                                  I32P, F32P, c_long], c_long)
    _DECLARED = True
    return L


def i32_array(values) -> ctypes.Array:
    return (c_int32 * max(1, len(values)))(*values)


def f32_array(values) -> ctypes.Array:
    return (c_float * max(1, len(values)))(*values)
