"""Refcounted paged-KV block allocator policy (dense ids, LIFO recycle, copy-on-write sharing), backed by the
C++ host library. Behavioural parity: core-llm/src/paging.rs:42-127."""
from __future__ import annotations

from ._lib import lib


class OutOfBlocks(RuntimeError):
    pass


class BlockAllocator:
    def __init__(self, capacity: int | None = None):
        self._lib = lib()
        self._h = self._lib.swb_alloc_new(-1 if capacity is None else capacity)
        self.capacity = capacity

    def __del__(self):
        try:
            self._lib.swb_alloc_free(self._h)
        except Exception:
            pass

    def alloc(self) -> int:
        b = self._lib.swb_alloc_alloc(self._h)
        if b < 0:
            raise OutOfBlocks(f"KV block pool exhausted ({self.capacity} blocks)")
        return b

    def retain(self, block: int) -> None:
        if self._lib.swb_alloc_retain(self._h, block) != 0:
            raise ValueError(f"retain of free block {block}")

    def release(self, block: int) -> None:
        if self._lib.swb_alloc_release(self._h, block) != 0:
            raise ValueError(f"release of free block {block}")

    def refcount(self, block: int) -> int:
        return self._lib.swb_alloc_refcount(self._h, block)

    def live_blocks(self) -> int:
        return self._lib.swb_alloc_live(self._h)

    def shared_blocks(self) -> int:
        return self._lib.swb_alloc_shared(self._h)

    def peak_live_blocks(self) -> int:
        return self._lib.swb_alloc_peak(self._h)

    def free_blocks(self) -> int | None:
        return None if self.capacity is None else self.capacity - self.live_blocks()
