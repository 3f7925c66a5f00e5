"""SANA Linear-DiT and its deep-compression autoencoder decoder (parity: candle-gen-sana/src/transformer.rs,
dc_ae.rs, config.rs; checkpoint keys are the diffusers `SanaTransformer2DModel` / `AutoencoderDC` names).

Trunk: 1 x 1 patch embedding of a 32-channel latent (no positional embedding), per block
  * self-attention that is LINEAR in the token count: with phi = ReLU, out = (V phi(K)^T) phi(Q) / (sum_n phi(K)) phi(Q)
    per head (70 heads of 32), so cost is O(N d^2) instead of O(N^2 d);
  * softmax cross-attention over the 300 caption tokens (20 heads of 112, no mask);
  * a Mix-FFN on the token grid: 1 x 1 conv -> SiLU -> 3 x 3 depthwise conv -> gated (a * silu(g)) -> 1 x 1 conv;
modulated adaLN-single style: one linear of the timestep embedding gives 6 vectors shared by all blocks, each block adds
its own learned table. SANA-Sprint adds a guidance embedding to the timestep embedding and RMS norms on q / k.

DC-AE decoder (32x spatial compression): conv_in + channel-repeat shortcut, six stages from deep to shallow, each an
up block (nearest-2x + conv, plus a pixel-shuffle shortcut) followed by residual blocks (conv-SiLU-conv-channel RMS
norm) or EfficientViT blocks (multi-scale ReLU linear attention + GLU depthwise conv), then norm -> ReLU -> conv_out.

One implementation serves both backends: fp32 on CPU; on a CUDA device the 1 x 1 convolutions and linears are tcgen05
GEMMs over NHWC rows, the depthwise and 3 x 3 convolutions go through the framework's convolution call."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from . import nn_dual as nd


@dataclass
class SanaConfig:
    in_channels: int = 32
    out_channels: int = 32
    num_attention_heads: int = 70
    attention_head_dim: int = 32
    num_layers: int = 20
    num_cross_attention_heads: int = 20
    cross_attention_head_dim: int = 112
    caption_channels: int = 2304
    mlp_ratio: float = 2.5
    patch_size: int = 1
    norm_eps: float = 1e-6
    caption_norm_eps: float = 1e-5
    attn_qk_norm_eps: float = 1e-5
    attn_eps: float = 1e-15
    guidance_embeds: bool = False
    guidance_embeds_scale: float = 0.1
    qk_norm: bool = False

    @property
    def inner(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @property
    def ffn_hidden(self) -> int:
        return int(self.mlp_ratio * self.inner)

    @staticmethod
    def sprint() -> "SanaConfig":
        return SanaConfig(guidance_embeds=True, qk_norm=True)

    @staticmethod
    def from_json(j: dict) -> "SanaConfig":
        d = {k: j[k] for k in SanaConfig.__dataclass_fields__ if k in j and k != "qk_norm"}
        if "qk_norm" in j:
            d["qk_norm"] = bool(j["qk_norm"])
        return SanaConfig(**d)


@dataclass
class DcAeConfig:
    in_channels: int = 3
    latent_channels: int = 32
    attention_head_dim: int = 32
    block_out_channels: tuple[int, ...] = (128, 256, 512, 512, 1024, 1024)
    layers_per_block: tuple[int, ...] = (3, 3, 3, 3, 3, 3)
    block_types: tuple[str, ...] = ("res", "res", "res", "evit", "evit", "evit")
    qkv_multiscales: tuple[int, ...] = (5,)
    norm_eps: float = 1e-5
    attn_eps: float = 1e-15
    scaling_factor: float = 0.41407

    @property
    def compression(self) -> int:
        return 1 << (len(self.block_out_channels) - 1)


def random_sana_weights(cfg: SanaConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    D, Hf = cfg.inner, cfg.ffn_hidden
    p = cfg.patch_size
    w["patch_embed.proj.weight"], w["patch_embed.proj.bias"] = rn(D, cfg.in_channels, p, p) * std, rn(D) * std
    te = "time_embed." if cfg.guidance_embeds else "time_embed.emb."
    lin(w, te + "timestep_embedder.linear_1", D, 256, std)
    lin(w, te + "timestep_embedder.linear_2", D, D, std)
    if cfg.guidance_embeds:
        lin(w, "time_embed.guidance_embedder.linear_1", D, 256, std)
        lin(w, "time_embed.guidance_embedder.linear_2", D, D, std)
    lin(w, "time_embed.linear", 6 * D, D, std)
    lin(w, "caption_projection.linear_1", D, cfg.caption_channels, std)
    lin(w, "caption_projection.linear_2", D, D, std)
    w["caption_norm.weight"] = 1.0 + rn(D) * 0.1
    for i in range(cfg.num_layers):
        b = f"transformer_blocks.{i}"
        w[b + ".scale_shift_table"] = rn(6, D) * 0.1
        for a in ("attn1", "attn2"):
            for n in ("to_q", "to_k", "to_v"):
                lin(w, f"{b}.{a}.{n}", D, D, std, bias=(a == "attn2"))
            lin(w, f"{b}.{a}.to_out.0", D, D, std)
            if cfg.qk_norm:
                w[f"{b}.{a}.norm_q.weight"], w[f"{b}.{a}.norm_k.weight"] = 1.0 + rn(D) * 0.1, 1.0 + rn(D) * 0.1
        w[b + ".ff.conv_inverted.weight"], w[b + ".ff.conv_inverted.bias"] = rn(2 * Hf, D, 1, 1) * std, rn(2 * Hf) * std
        w[b + ".ff.conv_depth.weight"], w[b + ".ff.conv_depth.bias"] = rn(2 * Hf, 1, 3, 3) * 0.2, rn(2 * Hf) * std
        w[b + ".ff.conv_point.weight"] = rn(D, Hf, 1, 1) * std
    w["scale_shift_table"] = rn(2, D) * 0.1
    lin(w, "proj_out", p * p * cfg.out_channels, D, std)
    return w


def relu_linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, eps: float) -> torch.Tensor:
    """q, k, v [B, G, hd, N] with q, k already non-negative -> [B, G, hd, N] (fp32)."""
    q, k, v = q.float(), k.float(), v.float()
    num = (v @ k.transpose(-1, -2)) @ q
    den = k.sum(-1, keepdim=True).transpose(-1, -2) @ q
    return num / (den + eps)


def _conv1x1(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
    """1 x 1 convolution on NCHW through the dual-backend linear (a GEMM over NHWC rows)."""
    B, C, H, W = x.shape
    y = nd.linear(x.permute(0, 2, 3, 1).reshape(B * H * W, C), w.reshape(w.shape[0], -1), b)
    return y.reshape(B, H, W, -1).permute(0, 3, 1, 2)


def glu_mbconv(x: torch.Tensor, w: dict, p: str, hidden: int) -> torch.Tensor:
    h = F.silu(_conv1x1(x, w[p + ".conv_inverted.weight"], w.get(p + ".conv_inverted.bias")))
    h = F.conv2d(h, w[p + ".conv_depth.weight"], w.get(p + ".conv_depth.bias"), padding=1, groups=2 * hidden)
    a, g = h[:, :hidden], h[:, hidden:]
    return _conv1x1(a * F.silu(g), w[p + ".conv_point.weight"], None)


class SanaDiT:
    def __init__(self, cfg: SanaConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.bag = nd.WeightBag(weights, dtype, device)
        self.dtype, self.device = self.bag.dtype, self.bag.device

    def weight_bytes(self) -> int:
        return self.bag.nbytes()

    def _temb(self, t: torch.Tensor, name: str) -> torch.Tensor:
        e = nd.sinusoidal_embedding(t.to(self.device), 256).to(self.dtype)
        return self.bag.lin(self.bag.lin(e, name + ".linear_1", act="silu"), name + ".linear_2")

    def _qk(self, x: torch.Tensor, key: str) -> torch.Tensor:
        return nd.rms_norm(x, self.bag[key], self.cfg.attn_qk_norm_eps) if self.cfg.qk_norm else x

    def caption(self, caption: torch.Tensor) -> torch.Tensor:
        """[B, L, caption_channels] -> projected + normalised caption stream (independent of the timestep)."""
        c = self.bag.lin(self.bag.lin(caption.to(self.device, self.dtype), "caption_projection.linear_1", act="gelu_tanh"),
                         "caption_projection.linear_2")
        return nd.rms_norm(c, self.bag["caption_norm.weight"], self.cfg.caption_norm_eps)

    def forward_grad(self, latent: torch.Tensor, caption: torch.Tensor, timestep: torch.Tensor,
                     guidance: torch.Tensor | None = None, projected: bool = False) -> torch.Tensor:
        """latent [B, C, H, W]; caption [B, L, caption_channels] (or the output of `caption()` with projected=True);
        timestep [B] (sigma * 1000 for the flow model, the sCM time for Sprint); guidance [B] (Sprint: scale * 0.1)."""
        cfg, dev, dt = self.cfg, self.device, self.dtype
        D, p = cfg.inner, cfg.patch_size
        B, _, Hh, Ww = latent.shape
        ph, pw = Hh // p, Ww // p
        N = ph * pw
        x = F.conv2d(latent.to(dev, dt), self.bag["patch_embed.proj.weight"], self.bag["patch_embed.proj.bias"], stride=p)
        x = x.reshape(B, D, N).transpose(1, 2).contiguous()
        te = "time_embed." if cfg.guidance_embeds else "time_embed.emb."
        emb = self._temb(timestep, te + "timestep_embedder")
        if cfg.guidance_embeds and guidance is not None:
            emb = emb + self._temb(guidance, "time_embed.guidance_embedder")
        temb = self.bag.lin(F.silu(emb.float()).to(dt), "time_embed.linear").reshape(B, 6, D)
        cap = caption.to(dev, dt) if projected else self.caption(caption)
        H1, hd1 = cfg.num_attention_heads, cfg.attention_head_dim
        H2, hd2 = cfg.num_cross_attention_heads, cfg.cross_attention_head_dim
        for i in range(cfg.num_layers):
            b = f"transformer_blocks.{i}"
            m = (self.bag[b + ".scale_shift_table"].float()[None] + temb.float()).to(dt)
            sh1, sc1, g1, sh2, sc2, g2 = (m[:, j:j + 1] for j in range(6))
            h = nd.layer_norm(x, eps=cfg.norm_eps) * (1 + sc1) + sh1
            a = b + ".attn1."
            q = self._qk(self.bag.lin(h, a + "to_q"), a + "norm_q.weight")
            k = self._qk(self.bag.lin(h, a + "to_k"), a + "norm_k.weight")
            v = self.bag.lin(h, a + "to_v")
            hdn = lambda t: t.reshape(B, N, H1, hd1).permute(0, 2, 3, 1)       # noqa: E731
            o = relu_linear_attention(F.relu(hdn(q)), F.relu(hdn(k)), hdn(v), cfg.attn_eps)
            o = o.permute(0, 3, 1, 2).reshape(B, N, D).to(dt)
            x = x + g1 * self.bag.lin(o, a + "to_out.0")
            a = b + ".attn2."
            q = self._qk(self.bag.lin(x, a + "to_q"), a + "norm_q.weight").reshape(B, N, H2, hd2)
            k = self._qk(self.bag.lin(cap, a + "to_k"), a + "norm_k.weight").reshape(B, -1, H2, hd2)
            v = self.bag.lin(cap, a + "to_v").reshape(B, -1, H2, hd2)
            x = x + self.bag.lin(nd.attention(q, k, v), a + "to_out.0")
            h = nd.layer_norm(x, eps=cfg.norm_eps) * (1 + sc2) + sh2
            grid = h.reshape(B, ph, pw, D).permute(0, 3, 1, 2)
            ff = glu_mbconv(grid, self.bag.w, b + ".ff", cfg.ffn_hidden)
            x = x + g2 * ff.permute(0, 2, 3, 1).reshape(B, N, D)
        m = (self.bag["scale_shift_table"].float()[None] + emb.float()[:, None, :]).to(dt)
        out = self.bag.lin(nd.layer_norm(x, eps=cfg.norm_eps) * (1 + m[:, 1:2]) + m[:, 0:1], "proj_out")
        oc = cfg.out_channels
        return out.reshape(B, ph, pw, p, p, oc).permute(0, 5, 1, 3, 2, 4).reshape(B, oc, ph * p, pw * p)

    @torch.no_grad()
    def forward(self, latent, caption, timestep, guidance=None, projected=False):
        return self.forward_grad(latent, caption, timestep, guidance, projected)


# ---- DC-AE decoder --------------------------------------------------------------------------------------------------------
def random_dcae_weights(cfg: DcAeConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    rn, _ = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}

    def conv(name, o, i, k, bias=True, groups=1):
        w[name + ".weight"] = rn(o, i // groups, k, k) * (std * 4 / (k * (i // groups) ** 0.5))
        if bias:
            w[name + ".bias"] = rn(o) * 0.01

    def trms(name, c):
        w[name + ".weight"], w[name + ".bias"] = 1.0 + rn(c) * 0.1, rn(c) * 0.05

    chs, n = cfg.block_out_channels, len(cfg.block_out_channels)
    conv("decoder.conv_in", chs[-1], cfg.latent_channels, 3)
    for i in range(n):
        ch = chs[i]
        off = 0
        if i + 1 < n:
            conv(f"decoder.up_blocks.{i}.0.conv", ch, chs[i + 1], 3)
            off = 1
        for j in range(cfg.layers_per_block[i]):
            p = f"decoder.up_blocks.{i}.{j + off}"
            if cfg.block_types[i] == "res":
                conv(p + ".conv1", ch, ch, 3)
                conv(p + ".conv2", ch, ch, 3, bias=False)
                trms(p + ".norm", ch)
            else:
                heads = ch // cfg.attention_head_dim
                for nme in ("to_q", "to_k", "to_v"):
                    w[f"{p}.attn.{nme}.weight"] = rn(ch, ch) * std
                for s_i, ks in enumerate(cfg.qkv_multiscales):
                    conv(f"{p}.attn.to_qkv_multiscale.{s_i}.proj_in", 3 * ch, 3 * ch, ks, bias=False, groups=3 * ch)
                    conv(f"{p}.attn.to_qkv_multiscale.{s_i}.proj_out", 3 * ch, 3 * ch, 1, bias=False, groups=3 * heads)
                w[f"{p}.attn.to_out.weight"] = rn(ch, ch * (1 + len(cfg.qkv_multiscales))) * std
                trms(p + ".attn.norm_out", ch)
                conv(p + ".conv_out.conv_inverted", 8 * ch, ch, 1)
                conv(p + ".conv_out.conv_depth", 8 * ch, 8 * ch, 3, groups=8 * ch)
                conv(p + ".conv_out.conv_point", ch, 4 * ch, 1, bias=False)
                trms(p + ".conv_out.norm", ch)
    trms("decoder.norm_out", chs[0])
    conv("decoder.conv_out", cfg.in_channels, chs[0], 3)
    return w


class DcAeDecoder:
    def __init__(self, cfg: DcAeConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.bag = nd.WeightBag({k: v for k, v in weights.items() if k.startswith("decoder.")}, dtype, device)
        self.dtype, self.device = self.bag.dtype, self.bag.device

    def _trms(self, x, p):
        xf = x.float()
        y = xf / torch.sqrt(xf.pow(2).mean(1, keepdim=True) + self.cfg.norm_eps)
        return (y * self.bag[p + ".weight"].float().view(1, -1, 1, 1) + self.bag[p + ".bias"].float().view(1, -1, 1, 1)).to(x.dtype)

    def _conv(self, x, p, pad=1, groups=1):
        return F.conv2d(x, self.bag[p + ".weight"], self.bag.get(p + ".bias"), padding=pad, groups=groups)

    def _res(self, x, p):
        h = self._conv(F.silu(self._conv(x, p + ".conv1")), p + ".conv2")
        return self._trms(h, p + ".norm") + x

    def _evit(self, x, p):
        cfg = self.cfg
        B, C, H, W = x.shape
        hd = cfg.attention_head_dim
        heads = C // hd
        a = p + ".attn"
        qkv = torch.cat([_conv1x1(x, self.bag[f"{a}.{n}.weight"], None) for n in ("to_q", "to_k", "to_v")], 1)
        multi = [qkv]
        for s_i, ks in enumerate(cfg.qkv_multiscales):
            m = self._conv(qkv, f"{a}.to_qkv_multiscale.{s_i}.proj_in", pad=ks // 2, groups=3 * C)
            multi.append(self._conv(m, f"{a}.to_qkv_multiscale.{s_i}.proj_out", pad=0, groups=3 * heads))
        groups = heads * len(multi)
        hid = torch.cat(multi, 1).reshape(B, groups, 3 * hd, H * W)
        o = relu_linear_attention(F.relu(hid[:, :, :hd]), F.relu(hid[:, :, hd:2 * hd]), hid[:, :, 2 * hd:], cfg.attn_eps)
        o = _conv1x1(o.reshape(B, groups * hd, H, W).to(x.dtype), self.bag[a + ".to_out.weight"], None)
        x = self._trms(o, a + ".norm_out") + x
        c = p + ".conv_out"
        return self._trms(glu_mbconv(x, self.bag.w, c, 4 * C), c + ".norm") + x

    def _up(self, x, p, out_ch):
        B, C, H, W = x.shape
        up = self._conv(F.interpolate(x, scale_factor=2, mode="nearest"), p + ".conv")
        r = out_ch * 4 // C
        short = F.pixel_shuffle(x.repeat_interleave(r, dim=1), 2)
        return up + short

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        """[B, latent_channels, h, w] (already divided by scaling_factor) -> [B, 3, 32 h, 32 w]."""
        cfg = self.cfg
        chs, n = cfg.block_out_channels, len(cfg.block_out_channels)
        z = latent.to(self.device, self.dtype)
        h = self._conv(z, "decoder.conv_in") + z.repeat_interleave(chs[-1] // cfg.latent_channels, dim=1)
        for i in reversed(range(n)):
            off = 0
            if i + 1 < n:
                h = self._up(h, f"decoder.up_blocks.{i}.0", chs[i])
                off = 1
            for j in range(cfg.layers_per_block[i]):
                p = f"decoder.up_blocks.{i}.{j + off}"
                h = self._res(h, p) if cfg.block_types[i] == "res" else self._evit(h, p)
        return self._conv(F.relu(self._trms(h, "decoder.norm_out")), "decoder.conv_out")
