"""Sequence-parallel (Ulysses-style) attention plumbing for DiT blocks over peer memory.

Every rank owns S/P tokens of the joint sequence for all heads outside attention, and H/P heads for all S tokens
inside it. The two all-to-alls are not separate collectives:

  * `gemm_scatter`  the QKV projection's epilogue stores each 16-column chunk straight into the buffer of the rank
                    that owns its head (tile by tile, overlapped with the main loop of the next tile);
  * `attn_scatter`  the attention kernel's epilogue stores each output row straight into the buffer of the rank
                    that owns the token;
  * `barrier`       a one-CTA flag barrier between producer and consumer kernels (bounded waits).

The reference has no sequence parallelism (its only multi-GPU feature is layer-block placement,
candle-llm/src/models/llama.rs:321-343); `NcclSequenceParallel` is the library-collective baseline we compare with.
Buffers come from torch's symmetric memory; kernels use plain peer stores (no multicast loads)."""
from __future__ import annotations

import ctypes

import torch

from .._native import kernels
from ..ops.runtime import check, ptr, stream_ptr
from .comm import Communicator


class UlyssesContext:
    """Symmetric buffers for one (S, St, heads, hidden, mlp) problem. Token layout: the joint sequence is
    [txt (St) | img (S - St)]; rank r owns txt rows [r*St/P, (r+1)*St/P) and img rows likewise, stored locally as
    [txt_l | img_l]."""

    def __init__(self, comm: Communicator, S: int, St: int, heads: int, hidden: int, extra_cols: int):
        import torch.distributed._symmetric_memory as symm_mem

        P = comm.world
        assert heads % P == 0 and St % P == 0 and (S - St) % P == 0, "tokens and heads must divide the world size"
        self.comm, self.S, self.St, self.heads, self.hidden = comm, S, St, heads, hidden
        self.Hl = heads // P
        self.St_l, self.Si_l = St // P, (S - St) // P
        self.S_l = self.St_l + self.Si_l
        dev = comm.device
        self.qkv = symm_mem.empty((S, 3 * self.Hl * 128), dtype=torch.bfloat16, device=dev)
        self.attn = symm_mem.empty((self.S_l, hidden + extra_cols), dtype=torch.bfloat16, device=dev)
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=dev)
        self.flags.zero_()
        self._handles = [symm_mem.rendezvous(t, comm.group) for t in (self.qkv, self.attn, self.flags)]
        mk = lambda h: (ctypes.c_void_p * P)(*[int(p) for p in h.buffer_ptrs])   # noqa: E731
        self._qkv_ptrs, self._attn_ptrs, self._flag_ptrs = (mk(h) for h in self._handles)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.bytes_sent = 0
        torch.cuda.synchronize(dev)
        comm.barrier()

    def barrier(self) -> None:
        check(kernels().swb_peer_barrier(self._flag_ptrs, self.epoch.data_ptr(), self.comm.rank, self.comm.world,
                                         stream_ptr()), "swb_peer_barrier")

    def gemm_scatter(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, stream_kind: str) -> None:
        """a [T_local, K] @ w[3*heads*128, K]^T (+bias) -> head owners' `qkv` buffers. stream_kind: 'txt' (rows are this
        rank's text tokens), 'img' (image tokens) or 'joint' ([txt_l | img_l])."""
        r = self.comm.rank
        T = a.shape[0]
        if stream_kind == "txt":
            split, off0, off1 = T, r * self.St_l, 0
        elif stream_kind == "img":
            split, off0, off1 = T, self.St + r * self.Si_l, 0
        else:
            split, off0, off1 = self.St_l, r * self.St_l, self.St + r * self.Si_l - self.St_l
        assert a.stride(1) == 1 and w.is_contiguous() and w.shape[0] == 3 * self.heads * 128
        rc = kernels().swb_gemm_bf16_scatter(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), T, w.shape[0],
                                             a.shape[1], ptr(bias), 0, self._qkv_ptrs, self.comm.world, self.heads,
                                             split, off0, off1, stream_ptr())
        check(rc, "swb_gemm_bf16_scatter")
        self.bytes_sent += T * w.shape[0] * 2 * (self.comm.world - 1) // self.comm.world

    def attn_scatter(self, scale: float) -> None:
        """Attention of this rank's heads over all S tokens (reads `qkv`), rows returned to the token owners' `attn`
        buffers at columns [rank*Hl*128, (rank+1)*Hl*128)."""
        HlD = self.Hl * 128
        q = self.qkv
        rc = kernels().swb_attn_dense_scatter(q.data_ptr(), q.stride(0), 128, q[:, HlD:].data_ptr(),
                                              q[:, 2 * HlD:].data_ptr(), q.stride(0), 128, self._attn_ptrs,
                                              self.comm.world, self.attn.stride(0), self.comm.rank * HlD, self.St,
                                              self.St_l, self.Si_l, self.S, self.S, self.Hl, self.Hl, scale,
                                              stream_ptr())
        check(rc, "swb_attn_dense_scatter")
        self.bytes_sent += self.S * HlD * 2 * (self.comm.world - 1) // self.comm.world
