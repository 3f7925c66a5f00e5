"""Weight-only quantised linears on the sm_100a kernels: GGUF Q4_K / Q8_0 blocks and group-affine (MLX-style) 4 / 8
bit with 64-wide groups. `QuantWeight` keeps the packed bytes on the device; `linear_quant` runs the fused
dequant-GEMM for decode-sized token counts and expands to bf16 + dense GEMM above that."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .._native import kernels
from .gemm import gemm_bf16, gemm_workspace
from .runtime import check, ptr, require_cuda, stream_ptr

FORMATS = {"Q4_K": 0, "Q8_0": 1, "AFFINE4": 2, "AFFINE8": 3}
MAX_FUSED_TOKENS = 64


@dataclass
class QuantWeight:
    fmt: str
    packed: torch.Tensor                 # uint8, [N, row_bytes]
    n: int
    k: int
    scales: torch.Tensor | None = None   # bf16 [N, K/64] (affine formats)
    biases: torch.Tensor | None = None

    @property
    def nbytes(self) -> int:
        extra = 0 if self.scales is None else self.scales.numel() * 4
        return self.packed.numel() + extra

    def to(self, device) -> "QuantWeight":
        mv = lambda t: None if t is None else t.to(device)   # noqa: E731
        return QuantWeight(self.fmt, self.packed.to(device), self.n, self.k, mv(self.scales), mv(self.biases))


def quantize_weight(w: torch.Tensor, fmt: str) -> QuantWeight:
    """w: [N, K] float tensor (K a multiple of 256) -> packed weight on w's device."""
    N, K = w.shape
    assert K % 256 == 0, "quantised linears need K to be a multiple of 256"
    if fmt in ("Q4_K", "Q8_0"):
        from ..io import gguf_quants as gq

        x = w.detach().float().cpu().numpy()
        raw = gq.quantize_q4_k(x.reshape(-1)) if fmt == "Q4_K" else gq.quantize_q8_0(x.reshape(-1))
        packed = torch.from_numpy(np.ascontiguousarray(raw).view(np.uint8).reshape(N, -1).copy())
        return QuantWeight(fmt, packed.to(w.device), N, K)
    bits = 4 if fmt == "AFFINE4" else 8
    g = w.detach().float().reshape(N, K // 64, 64)
    lo, hi = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    scale = ((hi - lo) / (2 ** bits - 1)).clamp_min(1e-8).bfloat16().float()
    bias = lo.bfloat16().float()
    q = ((g - bias) / scale).round().clamp(0, 2 ** bits - 1).to(torch.int64).reshape(N, K)
    per = 32 // bits
    shifts = (torch.arange(per, device=w.device) * bits).view(1, 1, per)
    words = (q.view(N, K // per, per) << shifts).sum(-1).to(torch.int64)
    packed = (words & 0xFFFFFFFF).to(torch.uint32 if hasattr(torch, "uint32") else torch.int64)
    packed_u8 = packed.cpu().numpy().astype(np.uint32).view(np.uint8).reshape(N, -1)
    return QuantWeight(fmt, torch.from_numpy(packed_u8.copy()).to(w.device), N, K,
                       scale.reshape(N, K // 64).bfloat16().contiguous(), bias.reshape(N, K // 64).bfloat16().contiguous())


def dequantize_reference(qw: QuantWeight) -> torch.Tensor:
    """fp32 [N, K] on the CPU with plain numpy / torch math (the oracle for the kernels)."""
    if qw.fmt in ("Q4_K", "Q8_0"):
        from ..io import gguf_quants as gq

        raw = qw.packed.cpu().numpy().reshape(-1)
        return torch.from_numpy(gq.dequantize(raw, qw.fmt, qw.n * qw.k).reshape(qw.n, qw.k).astype(np.float32))
    bits = 4 if qw.fmt == "AFFINE4" else 8
    words = torch.from_numpy(qw.packed.cpu().numpy().view(np.uint32).astype(np.int64)).reshape(qw.n, -1)
    per = 32 // bits
    shifts = (torch.arange(per) * bits).view(1, 1, per)
    q = ((words[..., None] >> shifts) & (2 ** bits - 1)).reshape(qw.n, qw.k).float()
    s = qw.scales.float().cpu().repeat_interleave(64, 1)
    b = qw.biases.float().cpu().repeat_interleave(64, 1)
    return q * s + b


def dequantize(qw: QuantWeight) -> torch.Tensor:
    """bf16 [N, K] on the device (one kernel)."""
    require_cuda(qw.packed)
    out = torch.empty((qw.n, qw.k), dtype=torch.bfloat16, device=qw.packed.device)
    check(kernels().swb_dequant_rows(FORMATS[qw.fmt], qw.packed.data_ptr(), ptr(qw.scales), ptr(qw.biases),
                                     out.data_ptr(), qw.n, qw.k, stream_ptr()), "swb_dequant_rows")
    return out


def linear_quant(a: torch.Tensor, qw: QuantWeight, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
                 splits: int = 0) -> torch.Tensor:
    """a [T, K] bf16 -> [T, N] bf16."""
    require_cuda(a, qw.packed)
    T = a.shape[0]
    assert a.dtype == torch.bfloat16 and a.stride(1) == 1 and a.shape[1] == qw.k
    if T > MAX_FUSED_TOKENS:
        return gemm_bf16(a, dequantize(qw), bias=bias, out=out)
    if out is None:
        out = torch.empty((T, qw.n), dtype=torch.bfloat16, device=a.device)
    ws = gemm_workspace(a.device)
    rc = kernels().swb_gemm_quant(FORMATS[qw.fmt], a.data_ptr(), a.stride(0), qw.packed.data_ptr(), ptr(qw.scales),
                                  ptr(qw.biases), out.data_ptr(), out.stride(0), T, qw.n, qw.k, ptr(bias),
                                  ws.data_ptr(), ws.numel(), splits, stream_ptr())
    check(rc, "swb_gemm_quant")
    return out


def linear_any(a: torch.Tensor, w, bias: torch.Tensor | None = None, out: torch.Tensor | None = None, **kw
               ) -> torch.Tensor:
    """a @ w^T for a dense bf16 weight or a QuantWeight (the projections of a model may be either)."""
    if isinstance(w, QuantWeight):
        assert not kw or set(kw) <= {"out_dtype"} and kw.get("out_dtype") in (None, torch.bfloat16)
        return linear_quant(a, w, bias=bias, out=out)
    return gemm_bf16(a, w, bias=bias, out=out, **kw)


def _q8_0_torch(w: torch.Tensor) -> torch.Tensor:
    N, K = w.shape
    g = w.float().reshape(N, K // 32, 32)
    d = (g.abs().amax(-1, keepdim=True) / 127.0).half()
    inv = torch.where(d.float() > 0, 1.0 / d.float(), torch.zeros_like(d, dtype=torch.float32))
    q = (g * inv).round().clamp(-127, 127).to(torch.int8)
    out = torch.empty((N, K // 32, 34), dtype=torch.uint8, device=w.device)
    out[..., :2] = d.view(torch.uint8).reshape(N, K // 32, 2)
    out[..., 2:] = q.view(torch.uint8)
    return out.reshape(N, -1)


def _q4_k_torch(w: torch.Tensor) -> torch.Tensor:
    """Min/max Q4_K on the device: per 32-weight sub-block scale = (max - min) / 15 and offset = -min (clamped at 0),
    both quantised to 6 bits against the super-block's largest scale / offset (fp16 d / dmin)."""
    N, K = w.shape
    g = w.float().reshape(N, K // 256, 8, 32)
    lo = g.amin(-1).clamp_max(0.0)
    hi = g.amax(-1)
    scale = ((hi - lo) / 15.0).clamp_min(0.0)
    mn = -lo
    d = (scale.amax(-1, keepdim=True) / 63.0).half()
    dmin = (mn.amax(-1, keepdim=True) / 63.0).half()
    inv_d = torch.where(d.float() > 0, 1.0 / d.float(), torch.zeros_like(d, dtype=torch.float32))
    inv_dm = torch.where(dmin.float() > 0, 1.0 / dmin.float(), torch.zeros_like(dmin, dtype=torch.float32))
    sc = (scale * inv_d).round().clamp(0, 63).to(torch.int32)          # [N, B, 8]
    m = (mn * inv_dm).round().clamp(0, 63).to(torch.int32)
    eff_s = d.float() * sc.float()
    eff_m = dmin.float() * m.float()
    inv_s = torch.where(eff_s > 0, 1.0 / eff_s, torch.zeros_like(eff_s))
    q = ((g + eff_m[..., None]) * inv_s[..., None]).round().clamp(0, 15).to(torch.int32)   # [N, B, 8, 32]
    out = torch.empty((N, K // 256, 144), dtype=torch.uint8, device=w.device)
    out[..., 0:2] = d.view(torch.uint8).reshape(N, K // 256, 2)
    out[..., 2:4] = dmin.view(torch.uint8).reshape(N, K // 256, 2)
    s_lo, s_hi, m_lo, m_hi = sc[..., :4], sc[..., 4:], m[..., :4], m[..., 4:]
    out[..., 4:8] = (s_lo | ((s_hi >> 4) << 6)).to(torch.uint8)
    out[..., 8:12] = (m_lo | ((m_hi >> 4) << 6)).to(torch.uint8)
    out[..., 12:16] = ((s_hi & 0xF) | ((m_hi & 0xF) << 4)).to(torch.uint8)
    pairs = q.reshape(N, K // 256, 4, 2, 32)                            # pair p: sub-blocks 2p (low nibbles), 2p+1 (high)
    out[..., 16:] = (pairs[:, :, :, 0] | (pairs[:, :, :, 1] << 4)).to(torch.uint8).reshape(N, K // 256, 128)
    return out.reshape(N, -1)


def quantize_on_device(w: torch.Tensor, fmt: str) -> QuantWeight:
    """Quantise a bf16 / fp32 [N, K] tensor where it lives (used for quantise-on-load of whole models)."""
    N, K = w.shape
    assert K % 256 == 0
    if fmt == "Q8_0":
        return QuantWeight(fmt, _q8_0_torch(w).contiguous(), N, K)
    if fmt == "Q4_K":
        return QuantWeight(fmt, _q4_k_torch(w).contiguous(), N, K)
    return quantize_weight(w.float(), fmt)
