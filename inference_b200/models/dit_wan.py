"""Wan video DiT (parity: candle-gen-wan/src/transformer.rs, rope.rs, wan14b.rs; checkpoint keys are the diffusers
`WanTransformer3DModel` names).

Video latents [C, F, H, W] are patched (1, 2, 2) into tokens that carry a three-axis rotary position (frame, row,
column; the head's 128 dimensions split 44 / 42 / 42). Every block: adaLN-modulated self-attention over all tokens
(q and k RMS-normalised across the whole width before the head split), cross-attention onto the projected text (after
an affine LayerNorm, no gate), adaLN-modulated GELU-tanh feed-forward. The six modulation vectors of a block are a
learned table plus a projection of the timestep embedding shared by all blocks. The T2V-A14B model is two such
networks, the "high-noise" expert above a timestep boundary and the "low-noise" expert below it.

One implementation serves both backends: fp32 on the CPU oracle backend; bf16 on a CUDA device, where projections run
on the tcgen05 GEMM (`text_encoders.linear`) and both attentions on the head-dim-128 tcgen05 attention kernel."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .nn_dual import adapter_residual

from .dit_flux import rope_table, timestep_embedding
from .text_encoders import linear


@dataclass
class WanConfig:
    num_attention_heads: int = 40
    attention_head_dim: int = 128
    num_layers: int = 40
    ffn_dim: int = 13824
    in_channels: int = 16
    out_channels: int = 16
    text_dim: int = 4096
    freq_dim: int = 256
    patch_size: tuple[int, int, int] = (1, 2, 2)
    eps: float = 1e-6

    @property
    def dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @property
    def rope_axes(self) -> tuple[int, int, int]:
        d = self.attention_head_dim
        hw = 2 * (d // 6)
        return d - 2 * hw, hw, hw

    @staticmethod
    def from_json(j: dict) -> "WanConfig":
        d = {k: j[k] for k in WanConfig.__dataclass_fields__ if k in j}
        if "patch_size" in d:
            d["patch_size"] = tuple(d["patch_size"])
        return WanConfig(**d)


def random_wan_weights(cfg: WanConfig, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"
                       ) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device)      # noqa: E731
    w: dict[str, torch.Tensor] = {}
    D = cfg.dim

    def lin(name, o, i):
        w[name + ".weight"], w[name + ".bias"] = (rn(o, i) * std).to(dtype), (rn(o) * std).to(dtype)

    pt, ph, pw = cfg.patch_size
    w["patch_embedding.weight"] = (rn(D, cfg.in_channels, pt, ph, pw) * std).to(dtype)
    w["patch_embedding.bias"] = (rn(D) * std).to(dtype)
    lin("condition_embedder.time_embedder.linear_1", D, cfg.freq_dim)
    lin("condition_embedder.time_embedder.linear_2", D, D)
    lin("condition_embedder.time_proj", 6 * D, D)
    lin("condition_embedder.text_embedder.linear_1", D, cfg.text_dim)
    lin("condition_embedder.text_embedder.linear_2", D, D)
    for i in range(cfg.num_layers):
        p = f"blocks.{i}"
        w[p + ".scale_shift_table"] = (rn(1, 6, D) * std).to(dtype)
        for a in ("attn1", "attn2"):
            for n in ("to_q", "to_k", "to_v", "to_out.0"):
                lin(f"{p}.{a}.{n}", D, D)
            for n in ("norm_q", "norm_k"):
                w[f"{p}.{a}.{n}.weight"] = (1.0 + rn(D) * 0.1).to(dtype)
        w[p + ".norm2.weight"], w[p + ".norm2.bias"] = (1.0 + rn(D) * 0.1).to(dtype), (rn(D) * 0.1).to(dtype)
        lin(p + ".ffn.net.0.proj", cfg.ffn_dim, D)
        lin(p + ".ffn.net.2", D, cfg.ffn_dim)
    w["scale_shift_table"] = (rn(1, 2, D) * std).to(dtype)
    lin("proj_out", cfg.out_channels * pt * ph * pw, D)
    return w


def video_position_ids(f: int, h: int, w: int, device="cpu") -> torch.Tensor:
    """[f*h*w, 3] (frame, row, column) in token order."""
    ids = torch.zeros(f, h, w, 3, device=device)
    ids[..., 0] = torch.arange(f, device=device)[:, None, None]
    ids[..., 1] = torch.arange(h, device=device)[None, :, None]
    ids[..., 2] = torch.arange(w, device=device)[None, None, :]
    return ids.reshape(-1, 3)


def _rope_pairs(x, cos, sin):
    """x [B, S, heads, hd], cos / sin [S, hd / 2]: rotation of consecutive pairs."""
    x0, x1 = x[..., 0::2].float(), x[..., 1::2].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack((x0 * c - x1 * s, x1 * c + x0 * s), -1).flatten(-2).to(x.dtype)


class WanDiT:
    def __init__(self, cfg: WanConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = {k: v.to(device=self.device, dtype=dtype).contiguous() for k, v in weights.items()}
        self.w["patch_embedding.weight"] = self.w["patch_embedding.weight"].reshape(cfg.dim, -1).contiguous()
        self.lora = None

    def _lin(self, x, name):
        y = linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))
        if self.lora is not None and name in self.lora:
            y = y + adapter_residual(self.lora[name], x)
        return y

    def _ln(self, x):
        return F.layer_norm(x.float(), (x.shape[-1],), eps=self.cfg.eps)

    def _rms(self, x, name):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * self.w[name + ".weight"].float()).to(x.dtype)

    def _attend(self, q, k, v):
        """q [B, Sq, heads, 128], k / v [B, Skv, heads, 128] -> [B, Sq, heads * 128]."""
        if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128:
            from .. import ops

            return ops.dense_attention(q.contiguous(), k.contiguous(), v.contiguous(), scale=128 ** -0.5)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).reshape(q.shape[0], q.shape[1], -1)

    def _attention(self, x, ctx, p, rope):
        B, S, D = x.shape
        nh, hd = self.cfg.num_attention_heads, self.cfg.attention_head_dim
        q = self._rms(self._lin(x, p + ".to_q"), p + ".norm_q").view(B, S, nh, hd)
        k = self._rms(self._lin(ctx, p + ".to_k"), p + ".norm_k").view(B, ctx.shape[1], nh, hd)
        v = self._lin(ctx, p + ".to_v").view(B, ctx.shape[1], nh, hd)
        if rope is not None:
            q, k = _rope_pairs(q, *rope), _rope_pairs(k, *rope)
        return self._lin(self._attend(q, k, v), p + ".to_out.0")

    def patchify(self, z: torch.Tensor) -> torch.Tensor:
        """[B, C, F, H, W] -> [B, tokens, C * pt * ph * pw] in the patch convolution's weight order."""
        B, C, Fr, H, W = z.shape
        pt, ph, pw = self.cfg.patch_size
        x = z.reshape(B, C, Fr // pt, pt, H // ph, ph, W // pw, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, (Fr // pt) * (H // ph) * (W // pw), C * pt * ph * pw)

    def unpatchify(self, x: torch.Tensor, Fr: int, H: int, W: int) -> torch.Tensor:
        """[B, tokens, pt * ph * pw * C] (channel fastest) -> [B, C, F, H, W]."""
        B = x.shape[0]
        pt, ph, pw = self.cfg.patch_size
        x = x.reshape(B, Fr // pt, H // ph, W // pw, pt, ph, pw, -1).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(B, -1, Fr, H, W)

    def embed_text(self, context: torch.Tensor) -> torch.Tensor:
        """Encoder states [B, L, text_dim] -> the cross-attention context [B, L, dim] (independent of the timestep)."""
        t = "condition_embedder.text_embedder."
        c = context.to(self.device, self.dtype)
        return self._lin(F.gelu(self._lin(c, t + "linear_1").float(), approximate="tanh").to(self.dtype), t + "linear_2")

    def patch_embed_tokens(self, z: torch.Tensor) -> tuple[torch.Tensor, tuple[int, int, int]]:
        """Latents [B, C, F, H, W] -> (tokens [B, S, dim], the (frames, rows, columns) token grid)."""
        pt, ph, pw = self.cfg.patch_size
        _, _, Fr, H, W = z.shape
        return self._lin(self.patchify(z.to(self.device, self.dtype)), "patch_embedding"), (Fr // pt, H // ph, W // pw)

    def grid_rope(self, grid: tuple[int, int, int]) -> tuple[torch.Tensor, torch.Tensor]:
        return rope_table(video_position_ids(*grid, self.device), self.cfg.rope_axes, 10000.0)

    def _time(self, timestep, B):
        """timestep [B] -> (embedding [B, dim], the six per-block modulation vectors [B, 6, dim] in fp32)."""
        cfg, dt = self.cfg, self.dtype
        c = "condition_embedder."
        te = timestep_embedding(timestep.to(self.device).float(), cfg.freq_dim, time_factor=1.0).to(dt)
        temb = self._lin(F.silu(self._lin(te, c + "time_embedder.linear_1").float()).to(dt), c + "time_embedder.linear_2")
        return temb, self._lin(F.silu(temb.float()).to(dt), c + "time_proj").float().view(B, 6, cfg.dim)

    def _block(self, x, p, tproj, ctx, rope):
        """One transformer block with checkpoint prefix `p` (`blocks.<i>`, or a control branch's `vace_blocks.<j>`)."""
        cfg, dt = self.cfg, self.dtype
        sh1, sc1, g1, sh2, sc2, g2 = (self.w[p + ".scale_shift_table"].float() + tproj).unsqueeze(2).unbind(1)
        h = (self._ln(x) * (1 + sc1) + sh1).to(dt)
        x = (x.float() + self._attention(h, h, p + ".attn1", rope).float() * g1).to(dt)
        n2 = F.layer_norm(x.float(), (cfg.dim,), self.w[p + ".norm2.weight"].float(), self.w[p + ".norm2.bias"].float(),
                          cfg.eps).to(dt)
        x = x + self._attention(n2, ctx, p + ".attn2", None)
        h = (self._ln(x) * (1 + sc2) + sh2).to(dt)
        f = self._lin(F.gelu(self._lin(h, p + ".ffn.net.0.proj").float(), approximate="tanh").to(dt), p + ".ffn.net.2")
        return (x.float() + f.float() * g2).to(dt)

    def forward_tokens(self, x, timestep, ctx, rope, hints: dict | None = None):
        """The block stack and the output head on an already embedded token sequence: x [B, S, dim], timestep [B]
        (sigma * 1000), ctx = embed_text(...), rope (cos, sin) [S, head_dim / 2] -> [B, S, pt * ph * pw * C]. Packed
        conditioning (several clips on one token axis, each with its own rotary table) enters here
        (candle-gen-wan/src/transformer.rs `forward_packed`). `hints` maps a block index to a residual added after that
        block (control branches)."""
        cfg = self.cfg
        dev, dt = self.device, self.dtype
        temb, tproj = self._time(timestep, x.shape[0])
        for i in range(cfg.num_layers):
            x = self._block(x, f"blocks.{i}", tproj, ctx, rope)
            if hints is not None and i in hints:
                x = (x.float() + hints[i].float()).to(dt)
        shift, scale = (self.w["scale_shift_table"].float() + temb.float()[:, None]).unsqueeze(2).unbind(1)
        return self._lin((self._ln(x) * (1 + scale) + shift).to(dt), "proj_out")

    def forward_grad(self, z, timestep, context, embedded: bool = False):
        """z [B, C, F, H, W] latents, timestep [B] (sigma * 1000), context [B, L, text_dim] (or embed_text(...) with
        embedded=True) -> velocity [B, C, F, H, W]."""
        _, _, Fr, H, W = z.shape
        x, grid = self.patch_embed_tokens(z)
        ctx = context.to(self.device, self.dtype) if embedded else self.embed_text(context)
        return self.unpatchify(self.forward_tokens(x, timestep, ctx, self.grid_rope(grid)), Fr, H, W)

    @torch.no_grad()
    def forward(self, z, timestep, context, embedded: bool = False):
        return self.forward_grad(z, timestep, context, embedded)
