"""MLX group-affine packs ({weight uint32, scales, biases}) and their lossless GGML forms
(candle-gen/src/quant/repack.rs:54-345).

An MLX 4-bit group (w = scale * q + bias, q in 0..15, 64 or 32 columns per group) is exactly one or two GGML Q4_1
blocks (d = scale, m = bias as fp16, 32 codes, low nibbles hold the first 16 codes and high nibbles the next 16), so
the repack changes layout only - provided scale and bias are fp16-representable, which `f16_exact` checks. 8-bit
packs are dequantised on their exact grid."""
from __future__ import annotations

import torch

MLX_GROUP_SIZE = 64
Q4_1_BLOCK = 32
Q4_1_BLOCK_BYTES = 20


def mlx_packed_bits(wq_cols: int, scales_cols: int, group_size: int = MLX_GROUP_SIZE) -> int:
    """Bits per code, from the packed width and the number of groups."""
    return wq_cols * 32 // (scales_cols * group_size)


def f16_exact(x: float) -> bool:
    t = torch.tensor(x, dtype=torch.float32)
    return bool(t.half().float() == t)


def _check(wq, scales, biases, group_size: int, codes_per_word: int, what: str) -> tuple[int, int]:
    out_dim, wq_cols = wq.shape
    in_dim = scales.shape[1] * group_size
    if scales.shape[0] != out_dim or tuple(biases.shape) != tuple(scales.shape) or wq_cols * codes_per_word != in_dim:
        raise ValueError(f"not an MLX group-{group_size} {what} pack: wq {tuple(wq.shape)}, scales "
                         f"{tuple(scales.shape)}, biases {tuple(biases.shape)}")
    return out_dim, in_dim


def _words(wq: torch.Tensor) -> torch.Tensor:
    return wq.to(torch.int64) & 0xFFFFFFFF if wq.dtype != torch.uint32 else wq.to(torch.int64)


def unpack_mlx_codes(wq: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 codes [out, in]: code i of a word sits at bits [bits*i, bits*i + bits)."""
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int64) * bits
    codes = (_words(wq).unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return codes.reshape(wq.shape[0], -1).to(torch.uint8)


def _affine(codes: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int) -> torch.Tensor:
    out_dim, in_dim = codes.shape
    g = codes.float().reshape(out_dim, in_dim // group_size, group_size)
    return (g * scales.float().unsqueeze(-1) + biases.float().unsqueeze(-1)).reshape(out_dim, in_dim)


def dequant_mlx_q4_reference(wq, scales, biases, group_size: int = MLX_GROUP_SIZE) -> torch.Tensor:
    _check(wq, scales, biases, group_size, 8, "Q4")
    return _affine(unpack_mlx_codes(wq, 4), scales, biases, group_size)


def dequant_mlx_q8(wq, scales, biases, group_size: int = MLX_GROUP_SIZE) -> torch.Tensor:
    _check(wq, scales, biases, group_size, 4, "Q8")
    return _affine(unpack_mlx_codes(wq, 8), scales, biases, group_size)


def repack_mlx_q4_to_q4_1(wq, scales, biases, group_size: int = MLX_GROUP_SIZE) -> torch.Tensor:
    """GGML Q4_1 bytes, uint8 [out, in / 32 * 20]."""
    if group_size % Q4_1_BLOCK != 0:
        raise ValueError(f"MLX Q4 group_size {group_size} must be a multiple of the Q4_1 block ({Q4_1_BLOCK})")
    out_dim, in_dim = _check(wq, scales, biases, group_size, 8, "Q4")
    codes = unpack_mlx_codes(wq, 4).reshape(out_dim, in_dim // Q4_1_BLOCK, Q4_1_BLOCK)
    rep = group_size // Q4_1_BLOCK
    d = scales.float().half().repeat_interleave(rep, dim=1)
    m = biases.float().half().repeat_interleave(rep, dim=1)
    out = torch.empty((out_dim, in_dim // Q4_1_BLOCK, Q4_1_BLOCK_BYTES), dtype=torch.uint8)
    out[..., 0:2] = d.contiguous().view(torch.uint8).reshape(out_dim, -1, 2)
    out[..., 2:4] = m.contiguous().view(torch.uint8).reshape(out_dim, -1, 2)
    out[..., 4:] = codes[..., :16] | (codes[..., 16:] << 4)
    return out.reshape(out_dim, -1)


def pack_mlx_affine(weight: torch.Tensor, bits: int, group_size: int = MLX_GROUP_SIZE
                    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Min/max affine quantisation into the MLX layout: (uint32 words [out, in*bits/32], scales, biases fp32)."""
    if bits not in (4, 8):
        raise ValueError(f"pack_mlx_affine: bits must be 4 or 8 (got {bits})")
    out_dim, in_dim = weight.shape
    if in_dim % group_size != 0:
        raise ValueError(f"pack_mlx_affine: in dim {in_dim} not a multiple of group {group_size}")
    per = 32 // bits
    if group_size % per != 0:
        raise ValueError(f"pack_mlx_affine: group {group_size} must be a multiple of {per} for {bits}-bit packing")
    levels = float((1 << bits) - 1)
    g = weight.float().reshape(out_dim, in_dim // group_size, group_size)
    lo, hi = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    scale = (hi - lo) / levels
    q = torch.where(scale > 0, ((g - lo) / torch.where(scale > 0, scale, torch.ones_like(scale))).round()
                    .clamp(0, levels), torch.zeros_like(g)).to(torch.int64)
    q = q.reshape(out_dim, in_dim // per, per)
    shifts = torch.arange(per, dtype=torch.int64) * bits
    words = (q << shifts).sum(-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32).view(torch.uint32)
    return words, scale.squeeze(-1), lo.squeeze(-1)
