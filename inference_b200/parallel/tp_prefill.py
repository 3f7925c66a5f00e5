"""Sequence-parallel tensor parallelism for prefill-sized token counts, with both collectives of a layer half fused
into compute kernels over peer memory:

  row-parallel GEMM (o_proj / down)   its epilogue stores every partial-sum tile straight into the slot buffer of the
                                      rank that owns the token row (the scatter half of a reduce-scatter, tile by tile
                                      while the next tile's MMAs run);
  `reduce_norm_gather`                the owner sums the P slots in rank order, adds its residual shard, applies RMSNorm
                                      and stores the normed row into every rank's gathered buffer (the all-gather that
                                      feeds the next column-parallel GEMM);
  one-CTA barrier                     orders the gather stores before the consumer GEMM.

The residual stream lives sharded by rows ([ceil(T/P), H] per rank). The library baseline is all-reduce after each
row-parallel GEMM (`Communicator.all_reduce`)."""
from __future__ import annotations

import ctypes

import torch

from .._native import kernels
from ..ops.runtime import check, stream_ptr
from .comm import Communicator


class TpPrefillContext:
    def __init__(self, comm: Communicator, hidden: int, max_tokens: int):
        import torch.distributed._symmetric_memory as symm_mem

        P = comm.world
        self.comm, self.hidden, self.max_tokens = comm, hidden, max_tokens
        self.max_rows = (max_tokens + P - 1) // P
        dev = comm.device
        L = kernels()
        self.slots = symm_mem.empty((P * self.max_rows * hidden,), dtype=torch.bfloat16, device=dev)
        self.gather = symm_mem.empty((max_tokens, hidden), dtype=torch.bfloat16, device=dev)
        self.flags = symm_mem.empty((L.swb_comm_flag_words(),), dtype=torch.int32, device=dev)
        self.bar_flags = symm_mem.empty((64,), dtype=torch.int32, device=dev)
        self.flags.zero_()
        self.bar_flags.zero_()
        hs = [symm_mem.rendezvous(t, comm.group) for t in (self.slots, self.gather, self.flags, self.bar_flags)]
        mk = lambda h: (ctypes.c_void_p * P)(*[int(p) for p in h.buffer_ptrs])   # noqa: E731
        self._slot_ptrs, self._gather_ptrs, self._flag_ptrs, self._bar_ptrs = (mk(h) for h in hs)
        self._handles = hs
        self.epochs = torch.zeros(L.swb_comm_max_ctas(), dtype=torch.int32, device=dev)
        self.bar_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        comm.barrier()

    def rows_per_rank(self, T: int) -> int:
        return (T + self.comm.world - 1) // self.comm.world

    def my_rows(self, T: int) -> tuple[int, int]:
        """(first global row, number of rows) owned by this rank."""
        tl = self.rows_per_rank(T)
        lo = min(T, self.comm.rank * tl)
        return lo, max(0, min(T, lo + tl) - lo)

    def gemm_scatter_rows(self, a: torch.Tensor, w: torch.Tensor) -> None:
        """Partial sums of a[T, K] @ w[H, K]^T go to the row owners' slot buffers."""
        T = a.shape[0]
        assert T <= self.max_tokens and w.shape[0] == self.hidden and a.stride(1) == 1 and w.is_contiguous()
        rc = kernels().swb_gemm_bf16_scatter_rows(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), T, self.hidden,
                                                  a.shape[1], self._slot_ptrs, self.comm.world, self.comm.rank,
                                                  self.rows_per_rank(T), stream_ptr())
        check(rc, "swb_gemm_bf16_scatter_rows")
        self.comm.bytes_moved += T * self.hidden * 2 * (self.comm.world - 1) // self.comm.world

    def reduce_norm_gather(self, T: int, residual_local: torch.Tensor, weight: torch.Tensor, eps: float,
                           w_offset: float = 0.0, reduce: bool = True) -> torch.Tensor:
        """Returns the gathered normed activations [T, H] (valid after the trailing barrier, which this call issues)."""
        lo, n = self.my_rows(T)
        rc = kernels().swb_reduce_norm_gather(self.slots.data_ptr(), self.comm.world if reduce else 0,
                                              residual_local.data_ptr(), residual_local.stride(0), weight.data_ptr(),
                                              eps, w_offset, self._gather_ptrs, self.hidden, lo, n,
                                              self.rows_per_rank(T), self.hidden, self._flag_ptrs,
                                              self.epochs.data_ptr(), self.comm.rank, self.comm.world, stream_ptr())
        check(rc, "swb_reduce_norm_gather")
        check(kernels().swb_peer_barrier(self._bar_ptrs, self.bar_epoch.data_ptr(), self.comm.rank, self.comm.world,
                                         stream_ptr()), "swb_peer_barrier")
        self.comm.bytes_moved += n * self.hidden * 2 * (self.comm.world - 1)
        return self.gather[:T]
