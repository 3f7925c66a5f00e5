"""Dense bf16 GEMM on tcgen05 (replaces the reference's cuBLAS `linear`, candle-llm/src/primitives/nn.rs:14-19)."""
from __future__ import annotations

import torch

from .._native import kernels
from .runtime import check, ptr, require_cuda, stream_ptr

ACT = {None: 0, "none": 0, "silu": 1, "gelu_tanh": 2, "swiglu_pairs": 3, "geglu_pairs": 4}
_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
WORKSPACE_BYTES = 64 * 1024 + (96 << 20)


def gemm_workspace(device: torch.device, slot: int = 0) -> torch.Tensor:
    """Per-(device, slot) split-K scratch. Launches sharing a slot must be ordered on one stream."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, slot)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None,
              residual: torch.Tensor | None = None, act: str | None = None, out: torch.Tensor | None = None,
              out_dtype: torch.dtype = torch.bfloat16, mode: int = -1, block_n: int = 0, ctas: int = 0,
              workspace: torch.Tensor | None = None) -> torch.Tensor:
    """out[T, N] = act(a[T, K] @ w[N, K]^T + bias) + residual. a and w are bf16 with contiguous rows."""
    require_cuda(a, w)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1]
    assert a.stride(1) == 1 and w.stride(1) == 1
    T, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if ACT[act] >= 3 else N      # gated pairs halve the width
    if out is None:
        out = torch.empty((T, n_out), dtype=out_dtype, device=a.device)
    assert out.shape == (T, n_out) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (T, N) and residual.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
    if workspace is None:
        workspace = gemm_workspace(a.device)
    rc = kernels().swb_gemm_bf16(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
                                 T, N, K, ptr(bias), ptr(residual), residual.stride(0) if residual is not None else 0,
                                 ACT[act], 1 if out.dtype == torch.float32 else 0, workspace.data_ptr(),
                                 workspace.numel(), mode, block_n, ctas, stream_ptr())
    check(rc, "swb_gemm_bf16")
    return out


def gemm_bf16_grouped(a: torch.Tensor, w: torch.Tensor, tile_groups: torch.Tensor, *, act: str | None = None,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped GEMM (replaces the reference's per-expert serial matmuls, candle-llm/src/models/llama.rs:1415-1488).

    a [R, K] with R a multiple of 128; w [G, N, K]; tile_groups int32 [R / 128] on the device: rows
    128*i .. 128*i+127 of a use w[tile_groups[i]]; a negative entry skips the tile (output rows untouched)."""
    require_cuda(a, w, tile_groups)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and tile_groups.dtype == torch.int32
    assert a.dim() == 2 and w.dim() == 3 and w.is_contiguous() and a.stride(1) == 1 and a.shape[1] == w.shape[2]
    R, K = a.shape
    G, N, _ = w.shape
    assert R % 128 == 0 and tile_groups.numel() == R // 128 and tile_groups.is_contiguous()
    if out is None:
        out = torch.empty((R, N), dtype=torch.bfloat16, device=a.device)
    assert out.shape == (R, N) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    rc = kernels().swb_gemm_bf16_grouped(a.data_ptr(), a.stride(0), w.data_ptr(), K, G, tile_groups.data_ptr(),
                                         out.data_ptr(), out.stride(0), R, N, K, ACT[act], stream_ptr())
    check(rc, "swb_gemm_bf16_grouped")
    return out


SSQ_WORDS = 64      # one u64 accumulator per token (2^-24 fixed point)


def ssq_buffer(device: torch.device) -> torch.Tensor:
    """A zeroed per-token sum-of-squares accumulator for a folded-RMSNorm chain (see gemm_bf16_normed)."""
    return torch.zeros(SSQ_WORDS, dtype=torch.int64, device=device)


def ssq_values(buf: torch.Tensor) -> torch.Tensor:
    """The accumulated sums of squares as fp32 [64]."""
    return buf.double().mul(2.0 ** -24).float()


def gemm_bf16_normed(a: torch.Tensor, w: torch.Tensor, *, out: torch.Tensor | None = None,
                     bias: torch.Tensor | None = None, residual: torch.Tensor | None = None, act: str | None = None,
                     ssq_in: torch.Tensor | None = None, ssq_out: torch.Tensor | None = None,
                     ssq_zero: torch.Tensor | None = None, norm_dim: int = 0, eps: float = 0.0) -> torch.Tensor:
    """One link of a folded-RMSNorm chain of decode GEMMs (T <= 64; see swb_gemm_bf16_normed).

    Consumer link (`ssq_in`): `a` is the un-normalised residual stream and `w` already carries the norm weight;
    the result is rmsnorm(a) @ w^T. Producer link (`ssq_out`): stores a @ w^T + residual (in place when out is
    residual) and adds the per-token sums of squares of what it stored to `ssq_out`, which must be zero at launch;
    `ssq_zero` is cleared by the launch (a chain alternates two accumulators: each producer clears the other one).
    Accumulators come from `ssq_buffer`."""
    require_cuda(a, w)
    T, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if ACT[act] >= 3 else N
    if out is None:
        out = torch.empty((T, n_out), dtype=torch.bfloat16, device=a.device)
    assert out.shape == (T, n_out) and out.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
    for b in (ssq_in, ssq_out, ssq_zero):
        assert b is None or (b.dtype == torch.int64 and b.numel() >= SSQ_WORDS and b.is_contiguous())
    rc = kernels().swb_gemm_bf16_normed(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                        out.stride(0), T, N, K, ptr(bias), ptr(residual),
                                        residual.stride(0) if residual is not None else 0, ACT[act], ptr(ssq_in),
                                        ptr(ssq_out), ptr(ssq_zero), norm_dim, eps, stream_ptr())
    check(rc, "swb_gemm_bf16_normed")
    return out


def gated_fused(T: int, N: int, K: int) -> bool:
    """True when linear_gated applies the activation inside the projection kernel for this shape."""
    return bool(kernels().swb_gemm_gated_supported(T, N, K))


def linear_gated(x: torch.Tensor, w_pairs: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """act(x W_gate^T) * (x W_up^T) for a gate-up weight whose rows are interleaved (gate_0, up_0, gate_1, ...).

    Decode-sized token counts apply the gated activation in the GEMM's epilogue (the reference runs the projection,
    a split and two elementwise kernels: candle-llm models/llama.rs:1386-1391); larger ones run the GEMM and the
    paired activation kernel."""
    from .llm import gated_act_mul

    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = w_pairs.shape[0]
    gelu = act in ("gelu", "gelu_tanh")
    if kernels().swb_gemm_gated_supported(T, N, K):
        y = gemm_bf16(x2, w_pairs, act="geglu_pairs" if gelu else "swiglu_pairs")
    else:
        y = gated_act_mul(gemm_bf16(x2, w_pairs), act, paired=True)
    return y.reshape(*x.shape[:-1], N // 2)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, **kw) -> torch.Tensor:
    """`x @ w^T (+ bias)` over the last dimension of x."""
    lead = x.shape[:-1]
    y = gemm_bf16(x.reshape(-1, x.shape[-1]), w, bias=bias, **kw)
    return y.reshape(*lead, w.shape[0])
