"""Device-resident paged KV pool and per-sequence block tables.

One allocation holds every layer's K and V blocks: [layers, 2, blocks, kv_heads_local, block_size, head_dim]
(sized for the 180 GB of a B200 up front instead of the reference's doubling growth,
candle-llm/src/primitives/paged_kv_cache.rs:101-140). Block ids are handed out by the refcounted
allocator policy (copy-on-write prefix sharing), so a block id is valid across all layers.
"""
from __future__ import annotations

import torch

from ..policy.paging import BlockAllocator


class PagedKvPool:
    def __init__(self, num_layers: int, num_blocks: int, kv_heads: int, head_dim: int, block_size: int = 16,
                 device: torch.device | str = "cuda", dtype: torch.dtype = torch.bfloat16):
        self.num_layers, self.num_blocks, self.block_size = num_layers, num_blocks, block_size
        self.kv_heads, self.head_dim = kv_heads, head_dim
        self.data = torch.zeros((num_layers, 2, num_blocks, kv_heads, block_size, head_dim), dtype=dtype,
                                device=device)
        self.allocator = BlockAllocator(num_blocks)

    @property
    def bytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    def copy_block(self, src: int, dst: int) -> None:
        """Copy-on-write: duplicate one block across all layers (K and V)."""
        self.data[:, :, dst].copy_(self.data[:, :, src])

    @staticmethod
    def blocks_for_budget(bytes_budget: int, num_layers: int, kv_heads: int, head_dim: int, block_size: int = 16,
                          elem: int = 2) -> int:
        per_block = num_layers * 2 * kv_heads * block_size * head_dim * elem
        return max(1, bytes_budget // per_block)


class PagedSequence:
    """Block table of one sequence over a pool: token i lives in blocks[i // bs] at offset i % bs."""

    _next_uid = 1

    def __init__(self, pool: PagedKvPool):
        self.pool = pool
        self.blocks: list[int] = []
        self.length = 0  # tokens whose K/V are (or are being) written
        self.uid = PagedSequence._next_uid  # never reused; with `epoch` it keys cached device block tables
        PagedSequence._next_uid += 1
        self.epoch = 0   # bumped whenever an already-published block id changes (COW unshare, truncate)

    @classmethod
    def seeded(cls, pool: PagedKvPool, blocks: list[int], length: int) -> "PagedSequence":
        """Share an existing prefix copy-on-write: retains the full blocks covering `length` tokens."""
        s = cls(pool)
        for b in blocks:
            pool.allocator.retain(b)
        s.blocks = list(blocks)
        s.length = length
        return s

    def reserve(self, n_tokens: int) -> list[int]:
        """Make room for n_tokens more tokens and return their flat cache slots (block * bs + offset)."""
        bs = self.pool.block_size
        slots = []
        for _ in range(n_tokens):
            bi, off = divmod(self.length, bs)
            if bi == len(self.blocks):
                self.blocks.append(self.pool.allocator.alloc())
            elif off == 0 or self.pool.allocator.refcount(self.blocks[bi]) > 1:
                # writing into a shared block: unshare it first (copy-on-write)
                if self.pool.allocator.refcount(self.blocks[bi]) > 1:
                    fresh = self.pool.allocator.alloc()
                    self.pool.copy_block(self.blocks[bi], fresh)
                    self.pool.allocator.release(self.blocks[bi])
                    self.blocks[bi] = fresh
                    self.epoch += 1
            slots.append(self.blocks[bi] * bs + off)
            self.length += 1
        return slots

    def truncate(self, length: int) -> None:
        """Roll back to `length` tokens (speculative rejection); frees blocks past the boundary."""
        bs = self.pool.block_size
        keep = (length + bs - 1) // bs
        for b in self.blocks[keep:]:
            self.pool.allocator.release(b)
        self.blocks = self.blocks[:keep]
        self.length = length
        self.epoch += 1

    def shareable_prefix_blocks(self, n_tokens: int) -> list[int]:
        """Blocks fully covered by the first n_tokens tokens (only whole blocks are shareable)."""
        return self.blocks[: n_tokens // self.pool.block_size]

    def release(self) -> None:
        for b in self.blocks:
            self.pool.allocator.release(b)
        self.blocks = []
        self.length = 0
