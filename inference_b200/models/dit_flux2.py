"""FLUX.2 MMDiT (parity: candle-gen-flux2/src/transformer.rs, pos_embed.rs, config.rs; checkpoint keys are the
diffusers `Flux2Transformer2DModel` names).

Differences from FLUX.1 that matter for execution: modulation is SHARED by all blocks of a kind (three linears per
step: image double-stream, text double-stream, single-stream, each (shift, scale, gate) sets), projections have no
biases, feed-forwards are SwiGLU (`linear_in` -> [a | b], silu(a) * b), a single block computes q / k / v and the
SwiGLU input with ONE projection (`to_qkv_mlp_proj`) and merges attention and MLP with one output projection, rotary
positions have four axes (t, h, w, layer) with text tokens indexed on the layer axis, and the timestep embedding gets
an optional guidance embedding added (dev). Latents are 128-channel tokens (32-channel VAE latents, 2 x 2 packed).

One implementation serves both backends (see nn_dual): fp32 on the CPU oracle backend, bf16 on a CUDA device with the
projections on the tcgen05 GEMM and the joint attention on the tcgen05 flash-attention kernel."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import nn_dual as nd

LN_EPS, RMS_EPS = 1e-6, 1e-5


@dataclass
class Flux2Config:
    num_double_layers: int = 8
    num_single_layers: int = 24
    num_heads: int = 32
    head_dim: int = 128
    in_channels: int = 128
    out_channels: int = 128
    joint_attention_dim: int = 12288
    mlp_ratio: float = 3.0
    timestep_channels: int = 256
    axes_dim: tuple[int, int, int, int] = (32, 32, 32, 32)
    rope_theta: float = 2000.0
    guidance_embed: bool = False

    @property
    def inner(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def mlp_hidden(self) -> int:
        return int(self.mlp_ratio * self.inner)

    @staticmethod
    def klein_9b() -> "Flux2Config":
        return Flux2Config()

    @staticmethod
    def dev() -> "Flux2Config":
        return Flux2Config(num_single_layers=48, num_heads=48, joint_attention_dim=15360, guidance_embed=True)

    @staticmethod
    def from_json(j: dict) -> "Flux2Config":
        alias = {"num_layers": "num_double_layers", "num_attention_heads": "num_heads", "attention_head_dim": "head_dim",
                 "axes_dims_rope": "axes_dim", "guidance_embeds": "guidance_embed"}
        d = {}
        for k, v in j.items():
            k = alias.get(k, k)
            if k in Flux2Config.__dataclass_fields__:
                d[k] = tuple(v) if k == "axes_dim" else v
        return Flux2Config(**d)


def random_flux2_weights(cfg: Flux2Config, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"):
    rn, lin = nd.randn_weights(seed, device)
    w: dict[str, torch.Tensor] = {}
    D, hd, M = cfg.inner, cfg.head_dim, cfg.mlp_hidden

    def L(name, o, i):
        lin(w, name, o, i, std, bias=False, dtype=dtype)

    def qk(p, names):
        for n in names:
            w[f"{p}.{n}.weight"] = (1.0 + rn(hd) * 0.1).to(dtype)

    L("x_embedder", D, cfg.in_channels)
    L("context_embedder", D, cfg.joint_attention_dim)
    for e in ("timestep_embedder",) + (("guidance_embedder",) if cfg.guidance_embed else ()):
        L(f"time_guidance_embed.{e}.linear_1", D, cfg.timestep_channels)
        L(f"time_guidance_embed.{e}.linear_2", D, D)
    L("double_stream_modulation_img.linear", 6 * D, D)
    L("double_stream_modulation_txt.linear", 6 * D, D)
    L("single_stream_modulation.linear", 3 * D, D)
    for i in range(cfg.num_double_layers):
        p = f"transformer_blocks.{i}"
        for n in ("to_q", "to_k", "to_v", "to_out.0", "add_q_proj", "add_k_proj", "add_v_proj", "to_add_out"):
            L(f"{p}.attn.{n}", D, D)
        qk(f"{p}.attn", ("norm_q", "norm_k", "norm_added_q", "norm_added_k"))
        for f in ("ff", "ff_context"):
            L(f"{p}.{f}.linear_in", 2 * M, D)
            L(f"{p}.{f}.linear_out", D, M)
    for i in range(cfg.num_single_layers):
        p = f"single_transformer_blocks.{i}.attn"
        L(f"{p}.to_qkv_mlp_proj", 3 * D + 2 * M, D)
        L(f"{p}.to_out", D, D + M)
        qk(p, ("norm_q", "norm_k"))
    L("norm_out.linear", 2 * D, D)
    L("proj_out", cfg.out_channels, D)
    return w


def grid_ids(lat_h: int, lat_w: int, t: int = 0) -> torch.Tensor:
    """[lat_h * lat_w, 4] (t, row, column, 0), row-major."""
    r = torch.arange(lat_h)[:, None].expand(lat_h, lat_w).reshape(-1)
    c = torch.arange(lat_w)[None, :].expand(lat_h, lat_w).reshape(-1)
    return torch.stack((torch.full_like(r, t), r, c, torch.zeros_like(r)), dim=1).float()


def text_ids(seq: int) -> torch.Tensor:
    """[seq, 4]: text tokens are numbered on the fourth (layer) axis."""
    z = torch.zeros(seq)
    return torch.stack((z, z, z, torch.arange(seq).float()), dim=1)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    a, b = x.chunk(2, dim=-1)
    return (F.silu(a.float()) * b.float()).to(x.dtype)


class Flux2DiT:
    def __init__(self, cfg: Flux2Config, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.bag = nd.WeightBag(weights, dtype, device)
        self.dtype, self.device = self.bag.dtype, self.bag.device
        self._rope_key, self._rope = None, None

    def weight_bytes(self) -> int:
        return self.bag.nbytes()

    def _sin_embed(self, scalar: torch.Tensor, name: str) -> torch.Tensor:
        e = nd.sinusoidal_embedding(scalar, self.cfg.timestep_channels).to(self.dtype)
        return self.bag.lin(self.bag.lin(e, name + ".linear_1", act="silu"), name + ".linear_2")

    def _mod(self, temb: torch.Tensor, name: str, sets: int):
        m = self.bag.lin(F.silu(temb.float()).to(self.dtype), name + ".linear")[:, None, :]
        c = m.chunk(3 * sets, dim=-1)
        return [(c[3 * i], c[3 * i + 1], c[3 * i + 2]) for i in range(sets)]       # (shift, scale, gate)

    def _heads(self, x: torch.Tensor, norm_key: str | None) -> torch.Tensor:
        B, S, _ = x.shape
        x = x.reshape(B, S, self.cfg.num_heads, self.cfg.head_dim)
        return nd.rms_norm(x, self.bag[norm_key], RMS_EPS) if norm_key else x

    def rope(self, img_ids: torch.Tensor, txt_ids: torch.Tensor):
        key = (tuple(img_ids.shape), tuple(txt_ids.shape), float(img_ids.sum()), float(txt_ids.sum()))
        if key != self._rope_key:
            cos, sin = nd.axis_rope_tables(torch.cat([txt_ids, img_ids], 0), self.cfg.axes_dim, self.cfg.rope_theta)
            self._rope_key, self._rope = key, (cos.to(self.device), sin.to(self.device))
        return self._rope

    def forward_grad(self, hidden: torch.Tensor, context: torch.Tensor, img_ids: torch.Tensor, txt_ids: torch.Tensor,
                     timestep: torch.Tensor, guidance: torch.Tensor | None = None) -> torch.Tensor:
        """hidden [B, S_img, in_channels] packed latent tokens, context [B, S_txt, joint_attention_dim], ids [S, 4],
        timestep [B] (sigma * 1000), guidance [B] (embedded scale; dev) -> velocity [B, S_img, out_channels]."""
        cfg, dev, dt = self.cfg, self.device, self.dtype
        D = cfg.inner
        temb = self._sin_embed(timestep.to(dev), "time_guidance_embed.timestep_embedder")
        if guidance is not None and "time_guidance_embed.guidance_embedder.linear_1.weight" in self.bag:
            temb = temb + self._sin_embed(guidance.to(dev) * 1000.0, "time_guidance_embed.guidance_embedder")
        img = self.bag.lin(hidden.to(dev, dt), "x_embedder")
        txt = self.bag.lin(context.to(dev, dt), "context_embedder")
        rope = self.rope(img_ids, txt_ids)
        im, tm = self._mod(temb, "double_stream_modulation_img", 2), self._mod(temb, "double_stream_modulation_txt", 2)
        n_txt = txt.shape[1]

        def modulate(x, scale, shift):
            return nd.layer_norm(x, eps=LN_EPS) * (1 + scale) + shift

        for i in range(cfg.num_double_layers):
            a = f"transformer_blocks.{i}.attn."
            ni, nt = modulate(img, im[0][1], im[0][0]), modulate(txt, tm[0][1], tm[0][0])
            q = torch.cat([self._heads(self.bag.lin(nt, a + "add_q_proj"), a + "norm_added_q.weight"),
                           self._heads(self.bag.lin(ni, a + "to_q"), a + "norm_q.weight")], 1)
            k = torch.cat([self._heads(self.bag.lin(nt, a + "add_k_proj"), a + "norm_added_k.weight"),
                           self._heads(self.bag.lin(ni, a + "to_k"), a + "norm_k.weight")], 1)
            v = torch.cat([self._heads(self.bag.lin(nt, a + "add_v_proj"), None),
                           self._heads(self.bag.lin(ni, a + "to_v"), None)], 1)
            o = nd.attention(nd.rope_interleaved(q, *rope), nd.rope_interleaved(k, *rope), v)
            img = img + self.bag.lin(o[:, n_txt:], a + "to_out.0") * im[0][2]
            txt = txt + self.bag.lin(o[:, :n_txt], a + "to_add_out") * tm[0][2]
            p = f"transformer_blocks.{i}."
            img = img + self.bag.lin(swiglu(self.bag.lin(modulate(img, im[1][1], im[1][0]), p + "ff.linear_in")),
                                     p + "ff.linear_out") * im[1][2]
            txt = txt + self.bag.lin(swiglu(self.bag.lin(modulate(txt, tm[1][1], tm[1][0]), p + "ff_context.linear_in")),
                                     p + "ff_context.linear_out") * tm[1][2]
        x = torch.cat([txt, img], 1)
        (shift, scale, gate), = self._mod(temb, "single_stream_modulation", 1)
        for i in range(cfg.num_single_layers):
            a = f"single_transformer_blocks.{i}.attn."
            proj = self.bag.lin(modulate(x, scale, shift), a + "to_qkv_mlp_proj")
            q, k, v, mlp = proj.split((D, D, D, proj.shape[-1] - 3 * D), dim=-1)
            o = nd.attention(nd.rope_interleaved(self._heads(q, a + "norm_q.weight"), *rope),
                             nd.rope_interleaved(self._heads(k, a + "norm_k.weight"), *rope), self._heads(v, None))
            x = x + self.bag.lin(torch.cat([o, swiglu(mlp)], -1), a + "to_out") * gate
        out = x[:, n_txt:]
        sc, sh = self.bag.lin(F.silu(temb.float()).to(dt), "norm_out.linear")[:, None, :].chunk(2, dim=-1)   # scale first
        return self.bag.lin(nd.layer_norm(out, eps=LN_EPS) * (1 + sc) + sh, "proj_out")

    @torch.no_grad()
    def forward(self, hidden, context, img_ids, txt_ids, timestep, guidance=None):
        return self.forward_grad(hidden, context, img_ids, txt_ids, timestep, guidance)


def vae_unpatchify(x: torch.Tensor) -> torch.Tensor:
    """[B, 4c, h, w] -> [B, c, 2h, 2w]; channel index = c * 4 + row-in-patch * 2 + column-in-patch."""
    B, C, h, w = x.shape
    return x.reshape(B, C // 4, 2, 2, h, w).permute(0, 1, 4, 2, 5, 3).reshape(B, C // 4, 2 * h, 2 * w)


def vae_patchify(x: torch.Tensor) -> torch.Tensor:
    B, c, h2, w2 = x.shape
    return x.reshape(B, c, h2 // 2, 2, w2 // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(B, 4 * c, h2 // 2, w2 // 2)
