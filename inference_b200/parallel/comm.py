"""Process-group bootstrap and the collective interface used by the models.

The reference has no communication backend at all (cross-device traffic is `Tensor::to_device` at
pipeline-shard boundaries, candle-llm/src/models/llama.rs:690-707); everything here is new. One process
drives one GPU; `torch.distributed` (NCCL on GPUs, gloo on CPU ranks) provides rendezvous, barriers and
the baseline collectives; the fused peer-memory kernels attach through `Communicator.fused`.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Any

import torch
import torch.distributed as dist


@dataclass
class Communicator:
    rank: int = 0
    world: int = 1
    group: Any = None
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    backend: str = "none"
    fused: Any = None          # parallel.symm.FusedCollectives when peer memory is available
    health: str = "healthy"    # healthy | degraded (NCCL fallback) | failed
    bytes_moved: int = 0

    @property
    def is_parallel(self) -> bool:
        return self.world > 1

    # ---- baseline collectives (library path; also the CPU / gloo path) -------------------------
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        if self.fused is not None and self.fused.can_all_reduce(t):
            return self.fused.all_reduce(t)
        dist.all_reduce(t, group=self.group)
        self.bytes_moved += t.numel() * t.element_size()
        return t

    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        self.bytes_moved += t.numel() * t.element_size() * (self.world - 1)
        return torch.cat(parts, dim=dim)

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over ranks, rank r keeps rows [r*n/P, (r+1)*n/P)."""
        if self.world == 1:
            return t
        out = torch.empty((t.shape[0] // self.world, *t.shape[1:]), dtype=t.dtype, device=t.device)
        if self.backend == "gloo":
            full = t.clone()
            dist.all_reduce(full, group=self.group)
            out.copy_(full.chunk(self.world, 0)[self.rank])
        else:
            dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
        return out

    def all_to_all(self, t: torch.Tensor, split_dim: int, cat_dim: int) -> torch.Tensor:
        """Split t into P chunks along split_dim, exchange, concatenate received chunks along cat_dim."""
        if self.world == 1:
            return t
        send = [c.contiguous() for c in t.chunk(self.world, dim=split_dim)]
        recv = [torch.empty_like(send[0]) for _ in range(self.world)]
        if self.backend == "gloo":
            for r in range(self.world):
                gathered = [torch.empty_like(send[0]) for _ in range(self.world)] if self.rank == r else None
                dist.gather(send[r], gathered, dst=r, group=self.group)
                if self.rank == r:
                    recv = gathered
        else:
            dist.all_to_all(recv, send, group=self.group)
        return torch.cat(recv, dim=cat_dim)

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world > 1:
            dist.broadcast(t, src=src, group=self.group)
        return t

    def barrier(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=self.device if self.backend == "nccl" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())


_DEFAULT: Communicator | None = None


def default_communicator() -> Communicator | None:
    """The communicator of this process's job (set by `init_distributed`), or None in a single-process run.
    Providers that can spread one request over the job's GPUs (sequence-parallel DiT rendering) pick it up at load
    time; every rank then issues the same `generate` call."""
    return _DEFAULT


def set_default_communicator(comm: Communicator | None) -> None:
    global _DEFAULT
    _DEFAULT = comm


def single(device: torch.device | str | None = None) -> Communicator:
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return Communicator(0, 1, None, torch.device(device), "none")


def init_distributed(backend: str | None = None, timeout_s: float = 600.0) -> Communicator:
    """Join the job described by RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    device = torch.device("cuda", local) if use_cuda and backend == "nccl" else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world == 1:
        return Communicator(0, 1, None, device, "none")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if not dist.is_initialized():
        kw = {"device_id": device} if device.type == "cuda" else {}
        dist.init_process_group(backend=backend, rank=rank, world_size=world, timeout=timedelta(seconds=timeout_s),
                                **kw)
    comm = Communicator(rank, world, dist.group.WORLD, device, backend)
    set_default_communicator(comm)
    return comm
