"""Token-granular longest-common-prefix index with LRU eviction (core-llm/src/prefix.rs:43-176).
Ids are never reused, so a backend can key cached KV blocks by PrefixId safely."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from ._lib import i32_array, lib


@dataclass(frozen=True)
class PrefixMatch:
    id: int
    matched_len: int


@dataclass(frozen=True)
class InsertOutcome:
    id: int
    evicted: list[int]


class PrefixIndex:
    def __init__(self, capacity: int):
        self._lib = lib()
        self.capacity = capacity
        self._h = self._lib.swb_prefix_new(capacity)

    def __del__(self):
        try:
            self._lib.swb_prefix_free(self._h)
        except Exception:
            pass

    def __len__(self) -> int:
        return self._lib.swb_prefix_len(self._h)

    def is_empty(self) -> bool:
        return len(self) == 0

    def contains(self, pid: int) -> bool:
        return bool(self._lib.swb_prefix_contains(self._h, pid))

    def longest_match(self, tokens: list[int]) -> PrefixMatch | None:
        pid, n = ctypes.c_uint64(), ctypes.c_long()
        if not self._lib.swb_prefix_longest_match(self._h, i32_array(tokens), len(tokens), ctypes.byref(pid),
                                                  ctypes.byref(n)):
            return None
        return PrefixMatch(pid.value, n.value)

    def insert(self, tokens: list[int]) -> InsertOutcome:
        pid = ctypes.c_uint64()
        cap = len(self) + 2
        ev = (ctypes.c_uint64 * cap)()
        k = self._lib.swb_prefix_insert(self._h, i32_array(tokens), len(tokens), ctypes.byref(pid), ev, cap)
        return InsertOutcome(pid.value, list(ev[:k]))
