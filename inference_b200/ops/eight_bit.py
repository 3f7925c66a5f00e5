"""8-bit linear layers: FP8 (E4M3) and INT8 with dynamic per-tensor activation scales, and the ConvRot regular
Hadamard rotation that flattens activation outliers before quantisation
(candle-gen/src/quant/cublaslt.rs:43-135, eight_bit_linear.rs:30-175, convrot.rs:50-99).

The reference multiplies through cuBLASLt. Here the multiply is the library's scaled GEMM on a CUDA device
(`torch._scaled_mm` for FP8, `torch._int_mm` for INT8 where the shape allows) and an exact emulation elsewhere
(codes converted to fp32, fp32 GEMM, scales applied after): both evaluate sum_k q_x q_w * s_x * s_w."""
from __future__ import annotations

import math
import sys

import torch

F8E4M3_MAX = 448.0
I8_MAX = 127.0
_TINY = sys.float_info.min if False else 1.1754943508222875e-38     # smallest normal fp32


def quantize_fp8(x: torch.Tensor) -> tuple[torch.Tensor, float]:
    """(E4M3 codes, scale) with scale = absmax / 448, at least the smallest normal fp32."""
    scale = max(float(x.detach().abs().max()) / F8E4M3_MAX, _TINY) if x.numel() else _TINY
    return (x.float() / scale).to(torch.float8_e4m3fn), scale


def quantize_int8(x: torch.Tensor) -> tuple[torch.Tensor, float]:
    scale = max(float(x.detach().abs().max()) / I8_MAX, _TINY) if x.numel() else _TINY
    return (x.float() / scale).round().clamp(-I8_MAX, I8_MAX).to(torch.int8), scale


def quantize_int8_per_channel(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per output row: (int8 codes [N, K], fp32 scales [N])."""
    scale = (w.detach().abs().amax(dim=1).float() / I8_MAX).clamp(min=_TINY)
    return (w.float() / scale[:, None]).round().clamp(-I8_MAX, I8_MAX).to(torch.int8), scale


def _flatten(x: torch.Tensor) -> tuple[torch.Tensor, tuple[int, ...]]:
    return x.reshape(-1, x.shape[-1]), tuple(x.shape[:-1])


class Fp8Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        self.w_fp8, self.scale_w = quantize_fp8(weight)
        self.bias = bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        flat, lead = _flatten(x)
        qx, sx = quantize_fp8(flat)
        M, K = flat.shape
        N = self.w_fp8.shape[0]
        if flat.is_cuda and K % 16 == 0 and N % 16 == 0:
            dev = flat.device
            y = torch._scaled_mm(qx, self.w_fp8.t(), scale_a=torch.tensor(sx, device=dev),
                                 scale_b=torch.tensor(self.scale_w, device=dev), out_dtype=torch.bfloat16).float()
        else:
            y = (qx.float() @ self.w_fp8.float().t()) * (sx * self.scale_w)
        y = y.reshape(*lead, N)
        return y + self.bias.to(y.dtype) if self.bias is not None else y

    __call__ = forward


class Int8Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, per_channel: bool = False):
        if per_channel:
            self.w_i8, self.scale_w = quantize_int8_per_channel(weight)
        else:
            self.w_i8, s = quantize_int8(weight)
            self.scale_w = torch.full((weight.shape[0],), s, dtype=torch.float32, device=weight.device)
        self.bias = bias

    @classmethod
    def from_per_channel_parts(cls, w_i8: torch.Tensor, scale_w: torch.Tensor, bias: torch.Tensor | None = None):
        if scale_w.numel() != w_i8.shape[0]:
            raise ValueError(f"Int8Linear.from_per_channel_parts: scale_w len {scale_w.numel()} != weight rows "
                             f"{w_i8.shape[0]}")
        self = cls.__new__(cls)
        self.w_i8, self.scale_w, self.bias = w_i8.to(torch.int8), scale_w.float(), bias
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        flat, lead = _flatten(x)
        qx, sx = quantize_int8(flat)
        M, K = flat.shape
        N = self.w_i8.shape[0]
        if flat.is_cuda and M > 16 and K % 8 == 0 and N % 8 == 0:
            acc = torch._int_mm(qx, self.w_i8.t()).float()
        else:
            acc = qx.float() @ self.w_i8.float().t()         # exact: |sum| < 2^24 for K <= 1040, else fp32-rounded
        y = (acc * sx * self.scale_w.to(acc.device)[None, :]).reshape(*lead, N)
        return y + self.bias.to(y.dtype) if self.bias is not None else y

    __call__ = forward


# ---- ConvRot ------------------------------------------------------------------------------------------------------------
_H4 = ((1.0, 1.0, 1.0, -1.0), (1.0, 1.0, -1.0, 1.0), (1.0, -1.0, 1.0, 1.0), (-1.0, 1.0, 1.0, 1.0))


def is_power_of_four(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0 and (n.bit_length() - 1) % 2 == 0


def regular_hadamard(group_size: int, device="cpu") -> torch.Tensor:
    """Symmetric orthogonal Hadamard matrix of order 4^k with constant row sums, built as Kronecker powers of the
    regular order-4 matrix and scaled by 1/sqrt(n): R = R^T = R^-1."""
    if not is_power_of_four(group_size):
        raise ValueError(f"ConvRot regular Hadamard order {group_size} is not a power of four (16, 64, 256, 1024, ...)")
    h4 = torch.tensor(_H4, dtype=torch.float32)
    h = torch.ones(1, 1)
    while h.shape[0] < group_size:
        h = torch.kron(h4, h)
    return (h / math.sqrt(group_size)).to(device)


def convrot_rotate(x: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    """Rotates each group of r.shape[0] consecutive features: rotating activations and weight columns by the same
    R leaves x W^T unchanged while spreading an outlier over its group."""
    n0 = r.shape[0]
    k = x.shape[-1]
    if k % n0 != 0:
        raise ValueError(f"ConvRot rotate: K ({k}) is not a multiple of group size ({n0})")
    return (x.float().reshape(-1, n0) @ r.float()).reshape(x.shape)
