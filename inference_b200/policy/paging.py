"""Refcounted paged-KV block allocator policy (dense ids, LIFO recycle, copy-on-write sharing).

Behavioural parity: core-llm/src/paging.rs:42-127 — `alloc` pops the most recently freed id or mints the
next dense id, `retain` adds a sharer, `release` frees at refcount 0, and the accounting exposes live,
shared and peak-live counts.
"""
from __future__ import annotations


class OutOfBlocks(RuntimeError):
    pass


class BlockAllocator:
    def __init__(self, capacity: int | None = None):
        self.capacity = capacity
        self._refs: list[int] = []
        self._free: list[int] = []
        self._live = 0
        self._peak = 0

    def alloc(self) -> int:
        if self._free:
            b = self._free.pop()
        else:
            if self.capacity is not None and len(self._refs) >= self.capacity:
                raise OutOfBlocks(f"KV block pool exhausted ({self.capacity} blocks)")
            b = len(self._refs)
            self._refs.append(0)
        self._refs[b] = 1
        self._live += 1
        self._peak = max(self._peak, self._live)
        return b

    def retain(self, block: int) -> None:
        if self._refs[block] <= 0:
            raise ValueError(f"retain of free block {block}")
        self._refs[block] += 1

    def release(self, block: int) -> None:
        if self._refs[block] <= 0:
            raise ValueError(f"release of free block {block}")
        self._refs[block] -= 1
        if self._refs[block] == 0:
            self._free.append(block)
            self._live -= 1

    def refcount(self, block: int) -> int:
        return self._refs[block] if 0 <= block < len(self._refs) else 0

    def live_blocks(self) -> int:
        return self._live

    def shared_blocks(self) -> int:
        return sum(1 for r in self._refs if r > 1)

    def peak_live_blocks(self) -> int:
        return self._peak

    def free_blocks(self) -> int | None:
        if self.capacity is None:
            return None
        return self.capacity - self._live
