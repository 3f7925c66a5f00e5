"""Symmetric (peer-mapped) memory and the fused collectives built on it.

Each rank allocates identical buffers through `torch.distributed._symmetric_memory` and exchanges handles once
at start-up; afterwards every rank holds the device pointers of all peers' buffers and kernels address them
directly over NVLink (plain peer loads / stores; no TMA multicast anywhere). `FusedCollectives` owns

  * two [max_tokens, hidden] bf16 exchange buffers (double buffered, see comm_allreduce.cu),
  * one flag pad per rank (epoch words, one row per CTA) and a local epoch counter array,

and offers `gemm_allreduce_rmsnorm`: the row-parallel GEMM writes its partial sums straight into the exchange
buffer and one kernel performs barrier + all-reduce + residual add + RMSNorm.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import ops
from .._native import kernels
from ..contracts.errors import CollectiveTimeout
from ..ops.runtime import check, ptr, stream_ptr
from .comm import Communicator


class FusedCollectives:
    def __init__(self, comm: Communicator, hidden: int, max_tokens: int = 256):
        import torch.distributed._symmetric_memory as symm_mem

        self.comm, self.hidden, self.max_tokens = comm, hidden, max_tokens
        dev = comm.device
        L = kernels()
        words = L.swb_comm_flag_words()
        self._bufs, self._buf_ptrs = [], []
        for _ in range(4):
            t = symm_mem.empty((max_tokens, hidden), dtype=torch.bfloat16, device=dev)
            h = symm_mem.rendezvous(t, comm.group)
            self._bufs.append(t)
            self._buf_ptrs.append((ctypes.c_void_p * comm.world)(*[int(p) for p in h.buffer_ptrs]))
        self._flags = symm_mem.empty((words,), dtype=torch.int32, device=dev)
        self._flags.zero_()
        fh = symm_mem.rendezvous(self._flags, comm.group)
        self._flag_ptrs = (ctypes.c_void_p * comm.world)(*[int(p) for p in fh.buffer_ptrs])
        self._epochs = torch.zeros(L.swb_comm_max_ctas(), dtype=torch.int32, device=dev)
        self._handles = [fh]
        # candidates of the distributed argmax: this rank's best (value, index in its vocabulary shard) per row
        self._am_vals = symm_mem.empty((max_tokens,), dtype=torch.float32, device=dev)
        self._am_ids = symm_mem.empty((max_tokens,), dtype=torch.int64, device=dev)
        vh, ih = symm_mem.rendezvous(self._am_vals, comm.group), symm_mem.rendezvous(self._am_ids, comm.group)
        self._am_val_ptrs = (ctypes.c_void_p * comm.world)(*[int(p) for p in vh.buffer_ptrs])
        self._am_id_ptrs = (ctypes.c_void_p * comm.world)(*[int(p) for p in ih.buffer_ptrs])
        self._handles += [vh, ih]
        # In-GEMM reduction of the row-parallel decode projections (GemmPeerReduce in gemm_tcgen05.cuh): two pairs of
        # line buffers (attention-out uses pair 0, MLP-down pair 1, so consecutive reductions alternate): slots
        # [world, chain_tokens, hidden / 8, 2 lines of 16 bytes] for the partial rows and results [chain_tokens,
        # hidden / 8, 2] for the rows a two-shot owner finishes; local launch counters per CTA.
        self.chain_tokens = min(64, max_tokens)
        ctas = L.swb_gemm_peer_max_ctas()
        self._pr_slots, self._pr_slot_ptrs, self._pr_results, self._pr_result_ptrs = [], [], [], []
        for _ in range(2):
            for shape, keep, ptrs in (((comm.world, self.chain_tokens, hidden // 8, 2, 4), self._pr_slots,
                                       self._pr_slot_ptrs),
                                      ((self.chain_tokens, hidden // 8, 2, 4), self._pr_results,
                                       self._pr_result_ptrs)):
                t = symm_mem.empty(shape, dtype=torch.int32, device=dev)
                t.zero_()
                h = symm_mem.rendezvous(t, comm.group)
                keep.append(t)
                ptrs.append((ctypes.c_void_p * comm.world)(*[int(p) for p in h.buffer_ptrs]))
                self._handles.append(h)
        self._pr_epochs = torch.zeros(ctas, dtype=torch.int32, device=dev)
        mode = os.environ.get("SWB_TP_REDUCE", "auto")
        self.reduce_mode = {"1": 1, "oneshot": 1, "2": 2, "twoshot": 2}.get(mode, 0)
        # Buffers 0/1 serve captured CUDA graphs (every capture starts at 0 and must contain an even number of
        # calls), buffers 2/3 serve eager launches, so consecutive collectives on the stream never reuse a buffer
        # that a peer may still be reading.
        self._next = {"graph": 0, "eager": 0}
        self._capturing = False
        torch.cuda.synchronize(dev)
        comm.barrier()

    # ---- capability checks used by Communicator -----------------------------------------------------------
    def can_all_reduce(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] == self.hidden and
                t.shape[0] <= self.max_tokens and t.stride(1) == 1)

    def exchange_buffer(self, tokens: int) -> tuple[torch.Tensor, int]:
        """The next exchange buffer (rows [0, tokens)) and its index; a GEMM writes its partial output here."""
        dom = "graph" if self._capturing else "eager"
        i = self._next[dom] + (0 if self._capturing else 2)
        self._next[dom] ^= 1
        return self._bufs[i][:tokens], i

    def begin_capture(self) -> None:
        self._capturing = True
        self._next["graph"] = 0

    def end_capture(self) -> None:
        self._capturing = False
        if self._next["graph"] != 0:
            raise RuntimeError("a captured step must contain an even number of fused collectives")

    def _launch(self, buf_index: int, T: int, residual, weight, eps, w_offset, out) -> None:
        rc = kernels().swb_allreduce_rmsnorm(self._buf_ptrs[buf_index], self._flag_ptrs, self._epochs.data_ptr(),
                                             self.comm.rank, self.comm.world, T, self.hidden, self.hidden,
                                             ptr(residual), residual.stride(0) if residual is not None else 0,
                                             ptr(weight), eps, w_offset, out.data_ptr(), out.stride(0), stream_ptr())
        check(rc, "swb_allreduce_rmsnorm")
        self.comm.bytes_moved += T * self.hidden * 2 * (self.comm.world - 1)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum over ranks of a [T <= max_tokens, hidden] bf16 tensor (copy into the exchange buffer)."""
        buf, i = self.exchange_buffer(t.shape[0])
        buf.copy_(t)
        self._launch(i, t.shape[0], None, None, 0.0, 0.0, t)
        return t

    def gemm_allreduce_rmsnorm(self, a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None,
                               norm_w: torch.Tensor | None, eps: float, w_offset: float = 0.0) -> torch.Tensor:
        """normed = rmsnorm(allreduce(a @ w^T) + residual) with the residual updated in place."""
        T = a.shape[0]
        buf, i = self.exchange_buffer(T)
        ops.linear_any(a, w, out=buf)
        out = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=a.device)
        self._launch(i, T, residual, norm_w, eps, w_offset, out)
        return out

    def peer_reduce_mode(self, tokens: int) -> int:
        """1 = one shot (every rank receives every partial), 2 = two shot (owners sum and send the finished rows).
        One shot moves (world - 1) x the row bytes per rank and has one hop; two shot moves about 2 x and has two."""
        if self.reduce_mode:
            return self.reduce_mode
        return 2 if self.comm.world > 2 and tokens * self.hidden * 4 * (self.comm.world - 1) > (1 << 20) else 1

    def gemm_peer_reduce(self, a: torch.Tensor, w: torch.Tensor, res: torch.Tensor, which: int,
                         ssq_out: torch.Tensor | None = None, ssq_zero: torch.Tensor | None = None,
                         cluster: int = 0) -> torch.Tensor:
        """res += sum over ranks of (a @ w^T), summed inside the GEMM's epilogue over peer memory (one kernel; no
        collective call). `which` (0: attention-out, 1: MLP-down) picks the line-buffer pair; consecutive calls on
        a stream must alternate it. ssq_out accumulates the per-token sums of squares of the new residual rows,
        ssq_zero is cleared (folded-norm chain, see ops.gemm_bf16_normed)."""
        T = a.shape[0]
        assert T <= self.chain_tokens and res.shape == (T, self.hidden) and res.stride(1) == 1
        a2 = a.reshape(T, -1)
        mode = self.peer_reduce_mode(T)
        rc = kernels().swb_gemm_bf16_peer_reduce(
            a2.data_ptr(), a2.stride(0), w.data_ptr(), w.stride(0), res.data_ptr(), res.stride(0), T, w.shape[0],
            a2.shape[1], res.data_ptr(), res.stride(0), ptr(ssq_out), ptr(ssq_zero), self._pr_slot_ptrs[which],
            self._pr_result_ptrs[which], self._pr_epochs.data_ptr(), self.chain_tokens, self.hidden, mode,
            self.comm.world, self.comm.rank, cluster, stream_ptr())
        check(rc, "swb_gemm_bf16_peer_reduce")
        self.comm.bytes_moved += T * self.hidden * 4 * ((self.comm.world - 1) if mode == 1 else 2)
        return res

    def argmax_vocab_parallel(self, local_logits: torch.Tensor, vocab_local: int) -> torch.Tensor:
        """Global greedy token ids [rows] from this rank's logits shard [rows <= max_tokens, vocab / world]: the local
        argmax kernel writes its (value, index) candidates into symmetric memory and one merge kernel (flag barrier +
        peer loads) picks the winner on every rank. Between two calls the step's all-reduce barriers separate a peer's
        reads from this rank's next writes, so one candidate buffer suffices."""
        rows = local_logits.shape[0]
        assert rows <= self.max_tokens
        ops.argmax(local_logits, out=self._am_ids[:rows], out_vals=self._am_vals[:rows])
        out = torch.empty(rows, dtype=torch.int64, device=local_logits.device)
        rc = kernels().swb_argmax_peer_merge(self._am_val_ptrs, self._am_id_ptrs, self._flag_ptrs,
                                             self._epochs.data_ptr(), self.comm.rank, self.comm.world, rows,
                                             vocab_local, out.data_ptr(), stream_ptr())
        check(rc, "swb_argmax_peer_merge")
        self.comm.bytes_moved += rows * 12 * (self.comm.world - 1)
        return out

    def check(self) -> None:
        st = ops.device_status()
        if st[0] == 3:
            kernels().swb_status_clear()
            self.comm.health = "degraded"
            raise CollectiveTimeout(f"peer wait timed out: where={st[1]} rank={st[2]} peer={st[3]}")


def attach_fused(comm: Communicator, hidden: int | None = None, max_tokens: int = 256) -> bool:
    """Enable the peer-memory collectives on `comm` when the world is parallel and symmetric memory works;
    otherwise leave the NCCL baseline in place (health = degraded). SWB_COMM=nccl forces the baseline."""
    if not comm.is_parallel or comm.backend != "nccl" or os.environ.get("SWB_COMM", "auto") == "nccl":
        return False
    from .health import FaultPlan

    if FaultPlan.from_env().denies("peer"):      # test seam: behave as if peer access were unavailable
        comm.fused = None
        comm.health = "degraded"
        comm.fused_error = "peer access denied by the fault plan"  # type: ignore[attr-defined]
        return False
    if hidden is None:
        comm._fused_pending = max_tokens  # type: ignore[attr-defined]  (created lazily by the model with its width)
        return True
    try:
        comm.fused = FusedCollectives(comm, hidden, max_tokens)
        return True
    except Exception as e:  # symmetric memory unavailable: keep NCCL
        comm.fused = None
        comm.health = "degraded"
        comm.fused_error = str(e)  # type: ignore[attr-defined]
        return False
