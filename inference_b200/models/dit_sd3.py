"""Stable Diffusion 3.5 MMDiT (parity: candle-gen-sd3/src/transformer.rs, config.rs; checkpoint keys are the diffusers
`SD3Transformer2DModel` names).

Image tokens (2x2 patches through a strided convolution, plus a centre crop of a stored 2-D position table) and
context tokens (CLIP-L/G features padded to the T5 width, then T5) run through joint blocks: each stream has its own
adaLN-Zero modulation, q/k/v projections with per-head RMSNorm and feed-forward; attention is over [image, context]
together; there is no rotary embedding. Blocks listed in `dual_attention_layers` (the Medium model) add a second,
image-only attention with its own modulation; the last block's context stream is "pre-only" (it feeds the attention and
stops). The conditioning vector is timestep embedding + pooled-text embedding.

One implementation serves both backends: fp32 on the CPU oracle backend, bf16 on a CUDA device where every projection
goes through the tcgen05 GEMM (`text_encoders.linear`) and attention through the tcgen05 attention kernel with the
64-wide heads zero-padded to its 128 (`ops.dense_attention_padded`)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .nn_dual import adapter_residual

from .dit_flux import timestep_embedding
from .text_encoders import linear


def _narrow_on_kernel() -> bool:
    from ..ops.attention import narrow_heads_on_kernel

    return narrow_heads_on_kernel()


@dataclass
class Sd3Config:
    in_channels: int = 16
    patch_size: int = 2
    pos_embed_max_size: int = 192
    num_attention_heads: int = 38
    attention_head_dim: int = 64
    num_layers: int = 38
    joint_attention_dim: int = 4096
    pooled_projection_dim: int = 2048
    qk_norm: bool = True
    dual_attention_layers: tuple[int, ...] = field(default_factory=tuple)

    @property
    def dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @property
    def patch_dim(self) -> int:
        return self.patch_size * self.patch_size * self.in_channels

    @staticmethod
    def large() -> "Sd3Config":
        return Sd3Config()

    @staticmethod
    def medium() -> "Sd3Config":
        return Sd3Config(pos_embed_max_size=384, num_attention_heads=24, num_layers=24,
                         dual_attention_layers=tuple(range(13)))

    @staticmethod
    def from_json(j: dict) -> "Sd3Config":
        d = {k: j[k] for k in Sd3Config.__dataclass_fields__ if k in j and k != "qk_norm"}
        if "dual_attention_layers" in d:
            d["dual_attention_layers"] = tuple(d["dual_attention_layers"])
        d["qk_norm"] = j.get("qk_norm", "rms_norm") is not None and j.get("qk_norm", "rms_norm") is not False
        return Sd3Config(**d)


def random_sd3_weights(cfg: Sd3Config, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"
                       ) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device)      # noqa: E731
    w: dict[str, torch.Tensor] = {}
    D = cfg.dim

    def lin(name, o, i):
        w[name + ".weight"], w[name + ".bias"] = (rn(o, i) * std).to(dtype), (rn(o) * std).to(dtype)

    def qknorm(p, names):
        if cfg.qk_norm:
            for n in names:
                w[f"{p}.{n}.weight"] = (1.0 + rn(cfg.attention_head_dim) * 0.1).to(dtype)

    w["pos_embed.proj.weight"] = (rn(D, cfg.in_channels, cfg.patch_size, cfg.patch_size) * std).to(dtype)
    w["pos_embed.proj.bias"] = (rn(D) * std).to(dtype)
    w["pos_embed.pos_embed"] = (rn(1, cfg.pos_embed_max_size ** 2, D) * 0.1).to(dtype)
    lin("time_text_embed.timestep_embedder.linear_1", D, 256)
    lin("time_text_embed.timestep_embedder.linear_2", D, D)
    lin("time_text_embed.text_embedder.linear_1", D, cfg.pooled_projection_dim)
    lin("time_text_embed.text_embedder.linear_2", D, D)
    lin("context_embedder", D, cfg.joint_attention_dim)
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}"
        last = i == cfg.num_layers - 1
        lin(f"{p}.norm1.linear", (9 if i in cfg.dual_attention_layers else 6) * D, D)
        lin(f"{p}.norm1_context.linear", (2 if last else 6) * D, D)
        for n in ("to_q", "to_k", "to_v", "to_out.0", "add_q_proj", "add_k_proj", "add_v_proj"):
            lin(f"{p}.attn.{n}", D, D)
        qknorm(f"{p}.attn", ("norm_q", "norm_k", "norm_added_q", "norm_added_k"))
        lin(f"{p}.ff.net.0.proj", 4 * D, D)
        lin(f"{p}.ff.net.2", D, 4 * D)
        if not last:
            lin(f"{p}.attn.to_add_out", D, D)
            lin(f"{p}.ff_context.net.0.proj", 4 * D, D)
            lin(f"{p}.ff_context.net.2", D, 4 * D)
        if i in cfg.dual_attention_layers:
            for n in ("to_q", "to_k", "to_v", "to_out.0"):
                lin(f"{p}.attn2.{n}", D, D)
            qknorm(f"{p}.attn2", ("norm_q", "norm_k"))
    lin("norm_out.linear", 2 * D, D)
    lin("proj_out", cfg.patch_dim, D)
    return w


def patchify(z: torch.Tensor, p: int = 2) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/p)(W/p), C*p*p] in the strided convolution's weight order (channel slowest)."""
    B, C, H, W = z.shape
    return z.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)


def unpatchify(x: torch.Tensor, h: int, w: int, p: int = 2) -> torch.Tensor:
    """[B, (h/p)(w/p), p*p*C] -> [B, C, h, w]; the output projection orders a patch as (row, column, channel)."""
    B, _, PD = x.shape
    C = PD // (p * p)
    return x.reshape(B, h // p, w // p, p, p, C).permute(0, 5, 1, 3, 2, 4).reshape(B, C, h, w)


class Sd3DiT:
    def __init__(self, cfg: Sd3Config, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = {k: v.to(device=self.device, dtype=dtype).contiguous() for k, v in weights.items()}
        self.w["pos_embed.proj.weight"] = self.w["pos_embed.proj.weight"].reshape(cfg.dim, -1).contiguous()
        self.lora = None

    def _lin(self, x, name):
        y = linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))
        if self.lora is not None and name in self.lora:
            y = y + adapter_residual(self.lora[name], x)
        return y

    def _ln(self, x):
        return F.layer_norm(x.float(), (x.shape[-1],), eps=1e-6).to(x.dtype)

    def _heads(self, x, norm_key):
        B, S, _ = x.shape
        x = x.view(B, S, self.cfg.num_attention_heads, self.cfg.attention_head_dim)
        wn = self.w.get(norm_key + ".weight")
        if wn is not None:
            xf = x.float()
            x = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()).to(x.dtype)
        return x.transpose(1, 2)

    def _sdpa(self, q, k, v):
        """q, k, v [B, heads, S, hd] -> [B, S, heads * hd]; on the device the zero-padded tcgen05 kernel."""
        B, _, S, D = q.shape
        if q.is_cuda and q.dtype == torch.bfloat16 and D <= 128 and D % 8 == 0 and _narrow_on_kernel():
            from .. import ops

            return ops.dense_attention_padded(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale=D ** -0.5)
        return F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, -1)

    def _ff(self, x, p):
        h = F.gelu(self._lin(x, p + ".net.0.proj").float(), approximate="tanh").to(x.dtype)
        return self._lin(h, p + ".net.2")

    def _block(self, i, x, c, sv):
        cfg = self.cfg
        p = f"transformer_blocks.{i}"
        last, dual = i == cfg.num_layers - 1, i in cfg.dual_attention_layers
        m = self._lin(sv, p + ".norm1.linear")[:, None, :].chunk(9 if dual else 6, -1)
        nx = self._ln(x)
        hx = nx * (1 + m[1]) + m[0]
        if last:
            scale, shift = self._lin(sv, p + ".norm1_context.linear")[:, None, :].chunk(2, -1)
            hc = self._ln(c) * (1 + scale) + shift
        else:
            mc = self._lin(sv, p + ".norm1_context.linear")[:, None, :].chunk(6, -1)
            hc = self._ln(c) * (1 + mc[1]) + mc[0]
        a = p + ".attn."
        n_img = x.shape[1]
        q = torch.cat([self._heads(self._lin(hx, a + "to_q"), a + "norm_q"),
                       self._heads(self._lin(hc, a + "add_q_proj"), a + "norm_added_q")], 2)
        k = torch.cat([self._heads(self._lin(hx, a + "to_k"), a + "norm_k"),
                       self._heads(self._lin(hc, a + "add_k_proj"), a + "norm_added_k")], 2)
        v = torch.cat([self._heads(self._lin(hx, a + "to_v"), "-"), self._heads(self._lin(hc, a + "add_v_proj"), "-")], 2)
        o = self._sdpa(q, k, v)
        x = x + m[2] * self._lin(o[:, :n_img], a + "to_out.0")
        if dual:
            h2 = nx * (1 + m[7]) + m[6]
            a2 = p + ".attn2."
            o2 = self._sdpa(self._heads(self._lin(h2, a2 + "to_q"), a2 + "norm_q"),
                            self._heads(self._lin(h2, a2 + "to_k"), a2 + "norm_k"),
                            self._heads(self._lin(h2, a2 + "to_v"), "-"))
            x = x + m[8] * self._lin(o2, a2 + "to_out.0")
        x = x + m[5] * self._ff(self._ln(x) * (1 + m[4]) + m[3], p + ".ff")
        if not last:
            c = c + mc[2] * self._lin(o[:, n_img:], a + "to_add_out")
            c = c + mc[5] * self._ff(self._ln(c) * (1 + mc[4]) + mc[3], p + ".ff_context")
        return x, c

    def forward_grad(self, z, timestep, context, pooled):
        """z [B, C, H, W] latent, timestep [B] (sigma * 1000), context [B, L, joint_attention_dim], pooled
        [B, pooled_projection_dim] -> [B, C, H, W]."""
        cfg = self.cfg
        B, _, H, W = z.shape
        p = cfg.patch_size
        h, w_ = H // p, W // p
        dev, dt = self.device, self.dtype
        x = self._lin(patchify(z.to(dev, dt), p), "pos_embed.proj")
        m = cfg.pos_embed_max_size
        top, left = (m - h) // 2, (m - w_) // 2
        pos = self.w["pos_embed.pos_embed"].view(m, m, cfg.dim)[top:top + h, left:left + w_].reshape(1, h * w_, cfg.dim)
        x = x + pos
        te = timestep_embedding(timestep.to(dev), 256, time_factor=1.0).to(dt)
        t = "time_text_embed."
        vec = self._lin(F.silu(self._lin(te, t + "timestep_embedder.linear_1").float()).to(dt), t + "timestep_embedder.linear_2")
        vec = vec + self._lin(F.silu(self._lin(pooled.to(dev, dt), t + "text_embedder.linear_1").float()).to(dt),
                              t + "text_embedder.linear_2")
        sv = F.silu(vec.float()).to(dt)
        c = self._lin(context.to(dev, dt), "context_embedder")
        for i in range(cfg.num_layers):
            x, c = self._block(i, x, c, sv)
        scale, shift = self._lin(sv, "norm_out.linear")[:, None, :].chunk(2, -1)
        out = self._lin(self._ln(x) * (1 + scale) + shift, "proj_out")
        return unpatchify(out, H, W, p)

    @torch.no_grad()
    def forward(self, z, timestep, context, pooled):
        return self.forward_grad(z, timestep, context, pooled)
