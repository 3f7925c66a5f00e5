"""Building blocks shared by the model families that have ONE implementation for both backends.

A model written on these helpers runs in fp32 on the CPU oracle backend (plain PyTorch: the numerics reference) and
in bf16 on a CUDA device, where the same calls route to this library's sm_100a kernels: every projection is the
tcgen05 GEMM (`ops.gemm_bf16`, bias / GELU / SiLU in its epilogue), attention over 128-wide heads is the tcgen05
flash-attention kernel (narrower heads are zero-padded onto it), RMSNorm is the vectorised norm kernel. What is left
(rotary rotation, modulation arithmetic, reshapes) is framework tensor code.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def on_device(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None, act: str | None = None) -> torch.Tensor:
    """x @ w^T + b with an optional activation ("silu", "gelu_tanh"; "gelu" = exact erf form) over the last dim."""
    if x.is_cuda and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.stride(1) == 1:
        from .. import ops

        lead = x.shape[:-1]
        fused = act if act in ("silu", "gelu_tanh") else None
        y = ops.gemm_bf16(x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous(), w, bias=b, act=fused)
        y = y.reshape(*lead, w.shape[0])
        if act == "gelu":
            y = F.gelu(y.float()).to(y.dtype)
        return y
    y = x.to(w.dtype) @ w.t()
    if b is not None:
        y = y + b
    if act == "silu":
        y = F.silu(y)
    elif act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif act == "gelu":
        y = F.gelu(y)
    return y


def rms_norm(x: torch.Tensor, w: torch.Tensor | None, eps: float = 1e-6, offset: float = 0.0) -> torch.Tensor:
    """x / rms(x) * (w + offset) over the last dim (fp32 statistics)."""
    if on_device(x) and w is not None and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        from .. import ops

        lead = x.shape
        return ops.rmsnorm(x.reshape(-1, lead[-1]).contiguous(), w, eps, w_offset=offset).reshape(lead)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * (w.float() + offset)
    return y.to(x.dtype)


def layer_norm(x: torch.Tensor, w: torch.Tensor | None = None, b: torch.Tensor | None = None, eps: float = 1e-6
               ) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float() if w is not None else None,
                        b.float() if b is not None else None, eps).to(x.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float | None = None,
              mask: torch.Tensor | None = None, causal: bool = False) -> torch.Tensor:
    """q [B, Sq, Hq, D], k / v [B, Skv, Hkv, D] (Hq a multiple of Hkv) -> [B, Sq, Hq * D].

    On the device, unmasked attention runs on the tcgen05 kernel (grouped-query heads natively, heads narrower than
    128 zero-padded); masked attention and the oracle backend use the framework's scaled-dot-product call."""
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else D ** -0.5
    if on_device(q) and mask is None and D <= 128 and D % 8 == 0 and (not causal or Sq == k.shape[1]):
        from .. import ops

        if D == 128 or (D == 64 and not causal):
            kc, vc = k.contiguous(), v.contiguous()
            return ops.dense_attention(q.contiguous(), kc, vc, scale=scale, causal=causal)
        if not causal:
            return ops.dense_attention_padded(q, k, v, scale=scale)
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if Hkv != Hq:
        kh = kh.repeat_interleave(Hq // Hkv, dim=1)
        vh = vh.repeat_interleave(Hq // Hkv, dim=1)
    o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, is_causal=causal and mask is None, scale=scale)
    return o.transpose(1, 2).reshape(B, Sq, Hq * D)


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotates adjacent pairs (x[2i], x[2i+1]) by the per-position angles. x [B, S, H, D]; cos / sin [S, D / 2]."""
    B, S, H, D = x.shape
    xr = x.float().reshape(B, S, H, D // 2, 2)
    c, s = cos.float().view(1, S, 1, D // 2), sin.float().view(1, S, 1, D // 2)
    xe, xo = xr[..., 0], xr[..., 1]
    return torch.stack((xe * c - xo * s, xe * s + xo * c), dim=-1).reshape(B, S, H, D).to(x.dtype)


def rope_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotates the pairs (x[i], x[i + D/2]) (the "rotate_half" convention). cos / sin [S, D / 2]."""
    B, S, H, D = x.shape
    xf = x.float()
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    c, s = cos.float().view(1, S, 1, D // 2), sin.float().view(1, S, 1, D // 2)
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


def axis_rope_tables(positions: torch.Tensor, axes: tuple[int, ...], theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """positions [S, len(axes)] (float) -> cos, sin [S, sum(axes) / 2]: per axis a block of axes[a] / 2 frequencies
    theta^(-2j / axes[a]), concatenated in axis order."""
    cols = []
    for a, d in enumerate(axes):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        cols.append(positions[:, a].double()[:, None] * inv[None, :])
    ang = torch.cat(cols, dim=1)
    return ang.cos().float(), ang.sin().float()


def sinusoidal_embedding(t: torch.Tensor, dim: int, *, max_period: float = 10000.0, cos_first: bool = True,
                         scale: float = 1.0) -> torch.Tensor:
    """[B] -> [B, dim]: frequencies max_period^(-i / (dim / 2)), angles t * scale * f."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = t.float()[:, None] * scale * freqs[None, :]
    parts = (ang.cos(), ang.sin()) if cos_first else (ang.sin(), ang.cos())
    return torch.cat(parts, dim=-1)


def patchify(z: torch.Tensor, p: int) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/p)(W/p), C*p*p], a patch ordered (channel, row, column)."""
    B, C, H, W = z.shape
    return z.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)


def unpatchify(x: torch.Tensor, ht: int, wt: int, p: int, c: int) -> torch.Tensor:
    """Inverse of patchify: [B, ht*wt, c*p*p] -> [B, c, ht*p, wt*p]."""
    B = x.shape[0]
    return x.reshape(B, ht, wt, c, p, p).permute(0, 3, 1, 4, 2, 5).reshape(B, c, ht * p, wt * p)


def adapter_residual(entry, x: torch.Tensor) -> torch.Tensor:
    """The additive branch of a trainable adapter on a linear layer. entry = (A [r, in], B [out, r], scale): LoRA,
    scale * B A x. entry = (w1 [a, c], w2_a [b, r], w2_b [r, d], scale): LoKr, scale * kron(w1, w2_a w2_b) x with
    out = a b and in = c d, applied factor by factor (never forming the dense delta)."""
    if len(entry) == 3:
        a, b, scale = entry
        return F.linear(F.linear(x, a), b) * scale
    w1, w2a, w2b, scale = entry
    (a, c), bd, d = w1.shape, w2a.shape[0], w2b.shape[1]
    lead, n = x.shape[:-1], x.numel() // x.shape[-1]
    t = (x.reshape(n * c, d) @ (w2a @ w2b).t().to(x.dtype)).reshape(n, c, bd)
    y = w1.to(x.dtype).reshape(1, a, c) @ t
    return y.reshape(*lead, a * bd) * scale


class WeightBag:
    """A flat name -> tensor map moved to one device / dtype, with the lookups a functional model needs."""

    def __init__(self, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu",
                 keep_fp32: tuple[str, ...] = ()):
        self.dtype, self.device = dtype, torch.device(device)
        self.w = {}
        for k, v in weights.items():
            dt = torch.float32 if (v.is_floating_point() and any(s in k for s in keep_fp32)) else \
                (dtype if v.is_floating_point() else v.dtype)
            self.w[k] = v.to(device=self.device, dtype=dt).contiguous()

    def __getitem__(self, k: str) -> torch.Tensor:
        return self.w[k]

    def get(self, k: str, default=None):
        return self.w.get(k, default)

    def __contains__(self, k: str) -> bool:
        return k in self.w

    def lin(self, x: torch.Tensor, name: str, act: str | None = None) -> torch.Tensor:
        return linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"), act)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.w.values())


def randn_weights(seed: int, device="cpu"):
    """(rn, lin) helpers for building random state dicts: rn(*shape) ~ N(0, 1); lin(dict, name, out, in, std, bias)."""
    g = torch.Generator(device=device).manual_seed(seed)

    def rn(*shape):
        return torch.randn(*shape, generator=g, device=device)

    def lin(w: dict, name: str, o: int, i: int, std: float = 0.05, bias: bool = True, dtype=torch.float32):
        w[name + ".weight"] = (rn(o, i) * std).to(dtype)
        if bias:
            w[name + ".bias"] = (rn(o) * std).to(dtype)

    return rn, lin
