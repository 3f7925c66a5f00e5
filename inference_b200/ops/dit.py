"""Wrappers for the media kernels: sampler axpy, GroupNorm(+SiLU), nearest upsample, row softmax, RGB8."""
from __future__ import annotations

import os

import torch

from .._native import kernels
from .runtime import check, ptr, require_cuda, stream_ptr


def axpy(a: float, x: torch.Tensor, b: float, y: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = a * x + b * y (the flow-matching Euler update is axpy(1, x, dt, v))."""
    require_cuda(x, y)
    assert x.shape == y.shape and x.dtype == y.dtype and x.is_contiguous() and y.is_contiguous()
    if out is None:
        out = torch.empty_like(x)
    rc = kernels().swb_axpy(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel(), a, b,
                            1 if x.dtype == torch.float32 else 0, stream_ptr())
    check(rc, "swb_axpy")
    return out


def groupnorm_nhwc(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, groups: int = 32, eps: float = 1e-6,
                   silu: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """x: [N, H, W, C] bf16 channels-last. GroupNorm with optional fused SiLU."""
    require_cuda(x)
    N, H, W, C = x.shape
    assert x.is_contiguous() and x.dtype == torch.bfloat16
    if out is None:
        out = torch.empty_like(x)
    stats = torch.empty((N, groups, 2), dtype=torch.float32, device=x.device)
    rc = kernels().swb_groupnorm(x.data_ptr(), stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), N,
                                 H * W, C, groups, eps, 1 if silu else 0, stream_ptr())
    check(rc, "swb_groupnorm")
    return out


def upsample2x_nhwc(x: torch.Tensor) -> torch.Tensor:
    require_cuda(x)
    N, H, W, C = x.shape
    out = torch.empty((N, 2 * H, 2 * W, C), dtype=x.dtype, device=x.device)
    check(kernels().swb_upsample2x(x.data_ptr(), out.data_ptr(), N, H, W, C, stream_ptr()), "swb_upsample2x")
    return out


def softmax_rows(scores: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """fp32 [R, C] -> bf16 probabilities softmax(scale * scores)."""
    require_cuda(scores)
    assert scores.dtype == torch.float32 and scores.stride(1) == 1
    out = torch.empty(scores.shape, dtype=torch.bfloat16, device=scores.device)
    check(kernels().swb_softmax_rows(scores.data_ptr(), out.data_ptr(), scores.shape[0], scores.shape[1],
                                     scores.stride(0), out.stride(0), scale, stream_ptr()), "swb_softmax_rows")
    return out


def rgb8_nhwc(x: torch.Tensor) -> torch.Tensor:
    """[N, H, W, C>=3] bf16 in [-1, 1] -> uint8 [N, H, W, 3] (round half to even)."""
    require_cuda(x)
    N, H, W, C = x.shape
    out = torch.empty((N, H, W, 3), dtype=torch.uint8, device=x.device)
    check(kernels().swb_rgb8(x.data_ptr(), out.data_ptr(), N * H * W, C, stream_ptr()), "swb_rgb8")
    return out


def conv3x3_supported(x: torch.Tensor) -> bool:
    """Shapes the implicit-GEMM convolution takes: 64-channel slabs, whole 128-pixel tiles that are a run of one image
    row or a stack of whole rows."""
    N, H, W, C = x.shape
    return C % 64 == 0 and (H * W) % 128 == 0 and (W % 128 == 0 or 128 % W == 0)


def conv3x3_nhwc(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                 act: str | None = None) -> torch.Tensor:
    """3x3 convolution (stride 1, zero padding 1) of x [N, H, W, C] bf16 with w [Cout, 9 * C] (columns ordered ky, kx,
    c) -> [N, H, W, Cout], bias / activation / residual [N, H, W, Cout] in the epilogue. Implicit GEMM on the tcgen05
    kernel: the nine shifted views of x are fetched by TMA, no patch matrix is materialised. Shapes outside
    `conv3x3_supported` take the patch-gather + GEMM path."""
    from .gemm import ACT, gemm_bf16

    require_cuda(x, w)
    N, H, W, C = x.shape
    Cout = w.shape[0]
    assert x.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == 9 * C and w.stride(1) == 1
    res2 = residual.reshape(N * H * W, Cout) if residual is not None else None
    if not conv3x3_supported(x) or os.environ.get("SWB_CONV3X3", "implicit") == "im2col":
        return gemm_bf16(im2col3x3_nhwc(x), w, bias=bias, residual=res2, act=act).view(N, H, W, Cout)
    out = torch.empty((N * H * W, Cout), dtype=torch.bfloat16, device=x.device)
    if res2 is not None:
        assert res2.dtype == torch.bfloat16 and res2.stride(1) == 1
    rc = kernels().swb_conv3x3_nhwc(x.data_ptr(), N, H, W, C, w.data_ptr(), w.stride(0), Cout, out.data_ptr(), out.stride(0),
                                    ptr(bias), ptr(res2), res2.stride(0) if res2 is not None else 0, ACT[act], stream_ptr())
    check(rc, "swb_conv3x3_nhwc")
    return out.view(N, H, W, Cout)


def im2col3x3_nhwc(x: torch.Tensor) -> torch.Tensor:
    """[N, H, W, C] bf16 -> [N*H*W, 9*C] patches (stride 1, zero padding 1), column order (kh, kw, c)."""
    require_cuda(x)
    N, H, W, C = x.shape
    assert x.is_contiguous() and x.dtype == torch.bfloat16
    out = torch.empty((N * H * W, 9 * C), dtype=x.dtype, device=x.device)
    check(kernels().swb_im2col3x3(x.data_ptr(), out.data_ptr(), N, H, W, C, stream_ptr()), "swb_im2col3x3")
    return out
