"""Stable Video Diffusion: the spatio-temporal UNet and the temporal-decoder autoencoder
(parity: candle-gen-svd/src/unet.rs, transformer.rs, vae.rs, conv3d.rs, embeddings.rs, scheduler.rs).

UNet: frames are a batch for every spatial layer ([B * F, C, H, W]); each residual block is a spatial ResNet followed by
a temporal ResNet (3x1x1 convolutions over the frame axis) blended by a learned sigmoid factor
(alpha * spatial + (1 - alpha) * temporal); each attention stage is a spatial transformer block followed by a temporal
block that attends across frames per pixel, with a sinusoidal frame-index embedding, blended the same way. Conditioning:
the CLIP image embedding as the single cross-attention token, and (fps - 1, motion bucket, noise augmentation) through
the added-time embedder. The input is the noisy latent concatenated with the conditioning-image latent (8 channels).

Autoencoder: a plain image encoder (the mode of the posterior is used) and a decoder whose residual blocks mix in a
temporal ResNet ((1 - alpha) * spatial + alpha * temporal: the opposite blend) and that ends with a 3-tap temporal
convolution over the decoded frames.

Runs in fp32 on both backends: the reference found half precision overflowing in the deep UNet and bf16 collapsing the
EDM denoise at sigma ~ 700."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import nn_dual as nd

CROSS_DIM = 1024


@dataclass
class SvdUnetConfig:
    in_channels: int = 8
    out_channels: int = 4
    block_out_channels: tuple[int, ...] = (320, 640, 1280, 1280)
    layers_per_block: int = 2
    cross_attention_dim: int = 1024
    num_attention_heads: tuple[int, ...] = (5, 10, 20, 20)
    transformer_layers_per_block: int = 1
    addition_time_embed_dim: int = 256
    projection_class_embeddings_input_dim: int = 768
    groups: int = 32

    @staticmethod
    def from_json(j: dict) -> "SvdUnetConfig":
        d = {k: (tuple(j[k]) if isinstance(j[k], list) else j[k]) for k in SvdUnetConfig.__dataclass_fields__ if k in j}
        return SvdUnetConfig(**d)


@dataclass
class SvdVaeConfig:
    in_channels: int = 3
    out_channels: int = 3
    latent_channels: int = 4
    block_out_channels: tuple[int, ...] = (128, 256, 512, 512)
    layers_per_block: int = 2
    scaling_factor: float = 0.18215
    groups: int = 32

    @staticmethod
    def from_json(j: dict) -> "SvdVaeConfig":
        d = {k: (tuple(j[k]) if isinstance(j[k], list) else j[k]) for k in SvdVaeConfig.__dataclass_fields__ if k in j}
        return SvdVaeConfig(**d)


def karras_sigmas(steps: int, sigma_min: float = 0.002, sigma_max: float = 700.0, rho: float = 7.0) -> list[float]:
    a, b = sigma_max ** (1 / rho), sigma_min ** (1 / rho)
    return [(a + (0.0 if steps == 1 else i / (steps - 1)) * (b - a)) ** rho for i in range(steps)] + [0.0]


class _Net:
    """Shared layer helpers over a flat weight dict."""

    def __init__(self, weights, dtype, device, groups):
        self.w = {k: v.to(device=device, dtype=dtype if v.is_floating_point() else v.dtype).contiguous() for k, v in weights.items()}
        self.dtype, self.device, self.groups = dtype, torch.device(device), groups

    def lin(self, x, n):
        return F.linear(x, self.w[n + ".weight"], self.w.get(n + ".bias"))

    def conv(self, x, n, stride=1, pad=1):
        return F.conv2d(x, self.w[n + ".weight"], self.w[n + ".bias"], stride=stride, padding=pad)

    def tconv(self, x, n):
        """[B, C, F, H, W] through a [O, I, k, 1, 1] kernel, zero-padded in time."""
        w = self.w[n + ".weight"]
        return F.conv3d(x, w, self.w[n + ".bias"], padding=((w.shape[2] - 1) // 2, 0, 0))

    def gn(self, x, n, eps):
        if x.dim() == 5:
            B, C, Fr, H, W = x.shape
            return F.group_norm(x, self.groups, self.w[n + ".weight"], self.w[n + ".bias"], eps)
        return F.group_norm(x, self.groups, self.w[n + ".weight"], self.w[n + ".bias"], eps)

    def ln(self, x, n):
        return F.layer_norm(x, (x.shape[-1],), self.w[n + ".weight"], self.w[n + ".bias"], 1e-5)

    def spatial_res(self, x, p, eps, temb=None):
        y = self.conv(F.silu(self.gn(x, p + ".norm1", eps)), p + ".conv1")
        if temb is not None:
            y = y + self.lin(F.silu(temb), p + ".time_emb_proj")[:, :, None, None]
        y = self.conv(F.silu(self.gn(y, p + ".norm2", eps)), p + ".conv2")
        return (self.conv(x, p + ".conv_shortcut", pad=0) if p + ".conv_shortcut.weight" in self.w else x) + y

    def temporal_res(self, x, p, eps, temb=None):
        y = self.tconv(F.silu(self.gn(x, p + ".norm1", eps)), p + ".conv1")
        if temb is not None:                                                   # [B, F, D] -> [B, C, F, 1, 1]
            y = y + self.lin(F.silu(temb), p + ".time_emb_proj").transpose(1, 2)[:, :, :, None, None]
        y = self.tconv(F.silu(self.gn(y, p + ".norm2", eps)), p + ".conv2")
        return (self.tconv(x, p + ".conv_shortcut") if p + ".conv_shortcut.weight" in self.w else x) + y

    def st_res(self, x, p, eps, frames, temb=None, temporal_weight_is_alpha=False):
        s = self.spatial_res(x, p + ".spatial_res_block", eps, temb)
        BF, C, H, W = s.shape
        B = BF // frames
        s5 = s.reshape(B, frames, C, H, W).permute(0, 2, 1, 3, 4)
        t5 = self.temporal_res(s5, p + ".temporal_res_block", eps, None if temb is None else temb.reshape(B, frames, -1))
        a = torch.sigmoid(self.w[p + ".time_mixer.mix_factor"])
        out = s5 * (1 - a) + t5 * a if temporal_weight_is_alpha else s5 * a + t5 * (1 - a)
        return out.permute(0, 2, 1, 3, 4).reshape(BF, C, H, W)


def timestep_embedding(x: torch.Tensor, dim: int) -> torch.Tensor:
    return nd.sinusoidal_embedding(x, dim, cos_first=True)


class SvdUnet(_Net):
    def __init__(self, cfg: SvdUnetConfig, weights, dtype=torch.float32, device="cpu"):
        super().__init__(weights, dtype, device, cfg.groups)
        self.cfg = cfg

    def _attn(self, x, ctx, p, heads):
        B, L, C = x.shape
        q = self.lin(x, p + ".to_q").reshape(B, L, heads, -1)
        k = self.lin(ctx, p + ".to_k").reshape(B, ctx.shape[1], heads, -1)
        v = self.lin(ctx, p + ".to_v").reshape(B, ctx.shape[1], heads, -1)
        return self.lin(nd.attention(q, k, v), p + ".to_out.0")

    def _geglu(self, x, p):
        a, b = self.lin(x, p + ".net.0.proj").chunk(2, dim=-1)
        return self.lin(a * F.gelu(b), p + ".net.2")

    def _transformer(self, x, ctx, p, heads, frames):
        BF, C, H, W = x.shape
        B, seq = BF // frames, H * W
        tctx = ctx.reshape(B, frames, *ctx.shape[1:])[:, :1].expand(B, seq, -1, -1).reshape(B * seq, *ctx.shape[1:])
        tok = self.lin(self.gn(x, p + ".norm", 1e-6).reshape(BF, C, seq).transpose(1, 2), p + ".proj_in")
        fidx = torch.arange(frames, device=self.device, dtype=torch.float32).repeat(B)
        pos = timestep_embedding(fidx, C).to(self.dtype)
        emb = self.lin(F.silu(self.lin(pos, p + ".time_pos_embed.linear_1")), p + ".time_pos_embed.linear_2")[:, None, :]
        a = torch.sigmoid(self.w[p + ".time_mixer.mix_factor"])
        for i in range(self.cfg.transformer_layers_per_block):
            b = f"{p}.transformer_blocks.{i}"
            n = self.ln(tok, b + ".norm1")
            tok = tok + self._attn(n, n, b + ".attn1", heads)
            tok = tok + self._attn(self.ln(tok, b + ".norm2"), ctx, b + ".attn2", heads)
            tok = tok + self._geglu(self.ln(tok, b + ".norm3"), b + ".ff")
            t = f"{p}.temporal_transformer_blocks.{i}"
            h = (tok + emb).reshape(B, frames, seq, C).transpose(1, 2).reshape(B * seq, frames, C)
            h = h + self._geglu(self.ln(h, t + ".norm_in"), t + ".ff_in")
            n = self.ln(h, t + ".norm1")
            h = h + self._attn(n, n, t + ".attn1", heads)
            h = h + self._attn(self.ln(h, t + ".norm2"), tctx, t + ".attn2", heads)
            h = h + self._geglu(self.ln(h, t + ".norm3"), t + ".ff")
            mix = h.reshape(B, seq, frames, C).transpose(1, 2).reshape(BF, seq, C)
            tok = tok * a + mix * (1 - a)
        return self.lin(tok, p + ".proj_out").transpose(1, 2).reshape(BF, C, H, W) + x

    @torch.no_grad()
    def forward(self, sample: torch.Tensor, timestep: float, image_embeds: torch.Tensor, added_time_ids: torch.Tensor) -> torch.Tensor:
        """sample [B, F, 8, h, w], image_embeds [B, ctx, 1024], added_time_ids [B, 3] -> [B, F, 4, h, w] (fp32)."""
        cfg = self.cfg
        boc, heads, n = cfg.block_out_channels, cfg.num_attention_heads, len(cfg.block_out_channels)
        B, Fr, Cin, H, W = sample.shape
        x = sample.to(self.device, self.dtype).reshape(B * Fr, Cin, H, W)
        ctx = image_embeds.to(self.device, self.dtype)
        t = torch.full((B,), float(timestep), device=self.device)
        emb = self.lin(F.silu(self.lin(timestep_embedding(t, boc[0]).to(self.dtype), "time_embedding.linear_1")), "time_embedding.linear_2")
        tid = timestep_embedding(added_time_ids.to(self.device).float().reshape(-1), cfg.addition_time_embed_dim).reshape(B, -1).to(self.dtype)
        emb = emb + self.lin(F.silu(self.lin(tid, "add_embedding.linear_1")), "add_embedding.linear_2")
        emb = emb.repeat_interleave(Fr, dim=0)
        ctx = ctx.repeat_interleave(Fr, dim=0)
        x = self.conv(x, "conv_in")
        skips = [x]
        for i in range(n):
            last = i == n - 1
            eps = 1e-5 if last else 1e-6
            for j in range(cfg.layers_per_block):
                x = self.st_res(x, f"down_blocks.{i}.resnets.{j}", eps, Fr, emb)
                if not last:
                    x = self._transformer(x, ctx, f"down_blocks.{i}.attentions.{j}", heads[i], Fr)
                skips.append(x)
            if not last:
                x = self.conv(x, f"down_blocks.{i}.downsamplers.0.conv", stride=2)
                skips.append(x)
        x = self.st_res(x, "mid_block.resnets.0", 1e-5, Fr, emb)
        x = self._transformer(x, ctx, "mid_block.attentions.0", heads[-1], Fr)
        x = self.st_res(x, "mid_block.resnets.1", 1e-5, Fr, emb)
        rheads = tuple(reversed(heads))
        for i in range(n):
            for j in range(cfg.layers_per_block + 1):
                x = self.st_res(torch.cat([x, skips.pop()], dim=1), f"up_blocks.{i}.resnets.{j}", 1e-5, Fr, emb)
                if i > 0:
                    x = self._transformer(x, ctx, f"up_blocks.{i}.attentions.{j}", rheads[i], Fr)
            if i < n - 1:
                x = self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"), f"up_blocks.{i}.upsamplers.0.conv")
        x = self.conv(F.silu(self.gn(x, "conv_norm_out", 1e-5)), "conv_out")
        return x.reshape(B, Fr, -1, H, W).float()


class SvdVae(_Net):
    def __init__(self, cfg: SvdVaeConfig, weights, dtype=torch.float32, device="cpu"):
        super().__init__(weights, dtype, device, cfg.groups)
        self.cfg = cfg

    def _attention(self, x, p):
        B, C, H, W = x.shape
        s = self.gn(x, p + ".group_norm", 1e-6).reshape(B, C, H * W).transpose(1, 2)
        q, k, v = self.lin(s, p + ".to_q"), self.lin(s, p + ".to_k"), self.lin(s, p + ".to_v")
        o = nd.attention(q[:, :, None], k[:, :, None], v[:, :, None])
        return x + self.lin(o, p + ".to_out.0").transpose(1, 2).reshape(B, C, H, W)

    @torch.no_grad()
    def encode_mode(self, image: torch.Tensor) -> torch.Tensor:
        """[B, 3, H, W] in [-1, 1] -> the posterior's mean [B, 4, H/8, W/8] (unscaled)."""
        cfg, e = self.cfg, "encoder."
        x = self.conv(image.to(self.device, self.dtype), e + "conv_in")
        n = len(cfg.block_out_channels)
        for i in range(n):
            for j in range(cfg.layers_per_block):
                x = self.spatial_res(x, f"{e}down_blocks.{i}.resnets.{j}", 1e-6)
            if i < n - 1:
                x = self.conv(F.pad(x, (0, 1, 0, 1)), f"{e}down_blocks.{i}.downsamplers.0.conv", stride=2, pad=0)
        x = self.spatial_res(x, e + "mid_block.resnets.0", 1e-6)
        x = self._attention(x, e + "mid_block.attentions.0")
        x = self.spatial_res(x, e + "mid_block.resnets.1", 1e-6)
        x = self.conv(F.silu(self.gn(x, e + "conv_norm_out", 1e-6)), e + "conv_out")
        m = F.conv2d(x, self.w["quant_conv.weight"], self.w["quant_conv.bias"])
        return m[:, : cfg.latent_channels]

    @torch.no_grad()
    def decode(self, z: torch.Tensor, frames: int) -> torch.Tensor:
        """[F, 4, h, w] (already divided by the scaling factor) -> [F, 3, 8h, 8w]."""
        cfg, d = self.cfg, "decoder."
        st = lambda x, p: self.st_res(x, p, 1e-6, frames, None, temporal_weight_is_alpha=True)      # noqa: E731
        x = self.conv(z.to(self.device, self.dtype), d + "conv_in")
        x = st(x, d + "mid_block.resnets.0")
        x = self._attention(x, d + "mid_block.attentions.0")
        x = st(x, d + "mid_block.resnets.1")
        n = len(cfg.block_out_channels)
        for i in range(n):
            for j in range(cfg.layers_per_block + 1):
                x = st(x, f"{d}up_blocks.{i}.resnets.{j}")
            if i < n - 1:
                x = self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"), f"{d}up_blocks.{i}.upsamplers.0.conv")
        x = self.conv(F.silu(self.gn(x, d + "conv_norm_out", 1e-6)), d + "conv_out")
        BF, C, H, W = x.shape
        x5 = x.reshape(BF // frames, frames, C, H, W).permute(0, 2, 1, 3, 4)
        return self.tconv(x5, d + "time_conv_out").permute(0, 2, 1, 3, 4).reshape(BF, C, H, W)


# ---- random weights -----------------------------------------------------------------------------------------------------
def _res_keys(w, rn, p, cin, cout, temb_dim, temporal: bool, std):
    def conv(n, o, i, k, kt=None):
        shape = (o, i, kt, 1, 1) if kt else (o, i, k, k)
        w[n + ".weight"] = rn(*shape) * std / math.sqrt(i * (kt or k * k) / 8)
        w[n + ".bias"] = rn(o) * 0.01

    def norm(n, c):
        w[n + ".weight"], w[n + ".bias"] = 1.0 + rn(c) * 0.05, rn(c) * 0.02

    s = p + ".spatial_res_block"
    norm(s + ".norm1", cin); conv(s + ".conv1", cout, cin, 3); norm(s + ".norm2", cout); conv(s + ".conv2", cout, cout, 3)      # noqa: E702
    if cin != cout:
        conv(s + ".conv_shortcut", cout, cin, 1)
    if temb_dim:
        w[s + ".time_emb_proj.weight"], w[s + ".time_emb_proj.bias"] = rn(cout, temb_dim) * std, rn(cout) * 0.01
    if temporal:
        t = p + ".temporal_res_block"
        norm(t + ".norm1", cout); conv(t + ".conv1", cout, cout, 0, 3); norm(t + ".norm2", cout); conv(t + ".conv2", cout, cout, 0, 3)      # noqa: E702
        if temb_dim:
            w[t + ".time_emb_proj.weight"], w[t + ".time_emb_proj.bias"] = rn(cout, temb_dim) * std, rn(cout) * 0.01
        w[p + ".time_mixer.mix_factor"] = rn(1) * 0.5


def random_svd_unet_weights(cfg: SvdUnetConfig, seed: int = 0, std: float = 0.1) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    boc, n = cfg.block_out_channels, len(cfg.block_out_channels)
    D = boc[0] * 4
    w["conv_in.weight"], w["conv_in.bias"] = rn(boc[0], cfg.in_channels, 3, 3) * std, rn(boc[0]) * 0.01
    lin(w, "time_embedding.linear_1", D, boc[0], std); lin(w, "time_embedding.linear_2", D, D, std)      # noqa: E702
    lin(w, "add_embedding.linear_1", D, cfg.projection_class_embeddings_input_dim, std); lin(w, "add_embedding.linear_2", D, D, std)      # noqa: E702

    def transformer(p, c):
        w[p + ".norm.weight"], w[p + ".norm.bias"] = 1.0 + rn(c) * 0.05, rn(c) * 0.02
        lin(w, p + ".proj_in", c, c, std); lin(w, p + ".proj_out", c, c, std)      # noqa: E702
        lin(w, p + ".time_pos_embed.linear_1", 4 * c, c, std); lin(w, p + ".time_pos_embed.linear_2", c, 4 * c, std)      # noqa: E702
        w[p + ".time_mixer.mix_factor"] = rn(1) * 0.5
        for i in range(cfg.transformer_layers_per_block):
            for b, temporal in ((f"{p}.transformer_blocks.{i}", False), (f"{p}.temporal_transformer_blocks.{i}", True)):
                names = ["norm1", "norm2", "norm3"] + (["norm_in"] if temporal else [])
                for nm in names:
                    w[f"{b}.{nm}.weight"], w[f"{b}.{nm}.bias"] = 1.0 + rn(c) * 0.05, rn(c) * 0.02
                for a, kv in (("attn1", c), ("attn2", cfg.cross_attention_dim)):
                    lin(w, f"{b}.{a}.to_q", c, c, std, bias=False); lin(w, f"{b}.{a}.to_k", c, kv, std, bias=False)      # noqa: E702
                    lin(w, f"{b}.{a}.to_v", c, kv, std, bias=False); lin(w, f"{b}.{a}.to_out.0", c, c, std)      # noqa: E702
                for ff in (["ff", "ff_in"] if temporal else ["ff"]):
                    lin(w, f"{b}.{ff}.net.0.proj", 8 * c, c, std); lin(w, f"{b}.{ff}.net.2", c, 4 * c, std)      # noqa: E702

    cin = boc[0]
    for i in range(n):
        for j in range(cfg.layers_per_block):
            _res_keys(w, rn, f"down_blocks.{i}.resnets.{j}", cin if j == 0 else boc[i], boc[i], D, True, std)
            if i < n - 1:
                transformer(f"down_blocks.{i}.attentions.{j}", boc[i])
        if i < n - 1:
            w[f"down_blocks.{i}.downsamplers.0.conv.weight"], w[f"down_blocks.{i}.downsamplers.0.conv.bias"] = rn(boc[i], boc[i], 3, 3) * std / 3, rn(boc[i]) * 0.01
        cin = boc[i]
    for k in (0, 1):
        _res_keys(w, rn, f"mid_block.resnets.{k}", boc[-1], boc[-1], D, True, std)
    transformer("mid_block.attentions.0", boc[-1])
    rb = tuple(reversed(boc))
    prev = rb[0]
    for i in range(n):
        out_c, in_c = rb[i], rb[min(i + 1, n - 1)]
        for j in range(cfg.layers_per_block + 1):
            skip = in_c if j == cfg.layers_per_block else out_c
            _res_keys(w, rn, f"up_blocks.{i}.resnets.{j}", (prev if j == 0 else out_c) + skip, out_c, D, True, std)
            if i > 0:
                transformer(f"up_blocks.{i}.attentions.{j}", out_c)
        if i < n - 1:
            w[f"up_blocks.{i}.upsamplers.0.conv.weight"], w[f"up_blocks.{i}.upsamplers.0.conv.bias"] = rn(out_c, out_c, 3, 3) * std / 3, rn(out_c) * 0.01
        prev = out_c
    w["conv_norm_out.weight"], w["conv_norm_out.bias"] = 1.0 + rn(boc[0]) * 0.05, rn(boc[0]) * 0.02
    w["conv_out.weight"], w["conv_out.bias"] = rn(cfg.out_channels, boc[0], 3, 3) * std / 3, rn(cfg.out_channels) * 0.01
    return w


def random_svd_vae_weights(cfg: SvdVaeConfig, seed: int = 0, std: float = 0.3) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    ch, n = cfg.block_out_channels, len(cfg.block_out_channels)

    def conv(name, o, i, k=3):
        w[name + ".weight"], w[name + ".bias"] = rn(o, i, k, k) * std / math.sqrt(i * k * k / 8), rn(o) * 0.01

    def norm(name, c):
        w[name + ".weight"], w[name + ".bias"] = 1.0 + rn(c) * 0.05, rn(c) * 0.02

    def attn(p, c):
        norm(p + ".group_norm", c)
        for nm in ("to_q", "to_k", "to_v", "to_out.0"):
            lin(w, f"{p}.{nm}", c, c, 0.05)

    def plain_res(p, cin, cout):
        tmp: dict = {}
        _res_keys(tmp, rn, "x", cin, cout, 0, False, std)
        for k, v in tmp.items():
            w[p + k[len("x.spatial_res_block"):]] = v

    e = "encoder."
    conv(e + "conv_in", ch[0], cfg.in_channels)
    cin = ch[0]
    for i in range(n):
        for j in range(cfg.layers_per_block):
            plain_res(f"{e}down_blocks.{i}.resnets.{j}", cin if j == 0 else ch[i], ch[i])
        if i < n - 1:
            conv(f"{e}down_blocks.{i}.downsamplers.0.conv", ch[i], ch[i])
        cin = ch[i]
    plain_res(e + "mid_block.resnets.0", ch[-1], ch[-1]); attn(e + "mid_block.attentions.0", ch[-1]); plain_res(e + "mid_block.resnets.1", ch[-1], ch[-1])      # noqa: E702
    norm(e + "conv_norm_out", ch[-1]); conv(e + "conv_out", 2 * cfg.latent_channels, ch[-1])      # noqa: E702
    conv("quant_conv", 2 * cfg.latent_channels, 2 * cfg.latent_channels, 1)
    d = "decoder."
    conv(d + "conv_in", ch[-1], cfg.latent_channels)
    for k in (0, 1):
        _res_keys(w, rn, f"{d}mid_block.resnets.{k}", ch[-1], ch[-1], 0, True, std)
    attn(d + "mid_block.attentions.0", ch[-1])
    rc = tuple(reversed(ch))
    prev = rc[0]
    for i in range(n):
        for j in range(cfg.layers_per_block + 1):
            _res_keys(w, rn, f"{d}up_blocks.{i}.resnets.{j}", prev if j == 0 else rc[i], rc[i], 0, True, std)
        if i < n - 1:
            conv(f"{d}up_blocks.{i}.upsamplers.0.conv", rc[i], rc[i])
        prev = rc[i]
    norm(d + "conv_norm_out", ch[0]); conv(d + "conv_out", cfg.out_channels, ch[0])      # noqa: E702
    w[d + "time_conv_out.weight"], w[d + "time_conv_out.bias"] = rn(cfg.out_channels, cfg.out_channels, 3, 1, 1) * 0.3, rn(cfg.out_channels) * 0.01
    return w
