"""Stream / pointer helpers and the device status word shared by every kernel wrapper."""
from __future__ import annotations

import ctypes

import torch

from .._native import kernels


class KernelError(RuntimeError):
    """A native launch returned an error code, or a bounded device-side wait ran out."""


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("sm_100a kernels need CUDA tensors; CPU execution goes through the fp32 oracle models")


def device_status() -> list[int]:
    """Synchronises and returns the 8-int status word (index 0 is the sticky error code)."""
    out = (ctypes.c_int * 8)()
    torch.cuda.synchronize()
    kernels().swb_status_read(out)
    return list(out)


def check_status() -> None:
    st = device_status()
    if st[0] != 0:
        kernels().swb_status_clear()
        raise KernelError(f"device-side wait timed out or failed: status={st}")
