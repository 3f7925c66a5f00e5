"""Qwen-Image autoencoder, decoder side, for single images (parity: candle-gen-qwen-image/src/vae.rs; checkpoint keys
are the diffusers `AutoencoderKLQwenImage` names).

The checkpoint is a video autoencoder with causal 3-D convolutions. A single image is one frame whose causal padding
is all zeros, so only the last temporal slice of every 3-D kernel ever meets data: each causal convolution becomes a
2-D convolution with `weight[:, :, -1]`. The norms are per-pixel L2 normalisations over channels
(x / ||x|| * sqrt(C) * gamma); the middle block has one single-head attention over pixels; three of the four up blocks
end in nearest 2x upsampling + a 3x3 convolution that halves the channels. Latents are stored normalised per channel
and are de-normalised (x * std + mean) before `post_quant_conv`."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

LATENTS_MEAN = (-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508, 0.4134, -0.0715, 0.5517, -0.3632,
                -0.1922, -0.9497, 0.2503, -0.2921)
LATENTS_STD = (2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743, 3.2687, 2.1526, 2.8652, 1.5579, 1.6382,
               1.1253, 2.8251, 1.916)
NORM_EPS = 1e-12


@dataclass
class QwenVaeConfig:
    base_dim: int = 96
    z_dim: int = 16
    dim_mult: tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2

    def up_plan(self) -> list[tuple[int, int, int | None]]:
        """(input channels, width, channels after the upsampler or None) for every up block, top first."""
        dims = [self.base_dim * m for m in (self.dim_mult[-1],) + tuple(reversed(self.dim_mult))]
        plan = []
        for i, (cin, width) in enumerate(zip(dims[:-1], dims[1:])):
            if i > 0:
                cin //= 2                       # the previous block's upsampler halved the channels
            plan.append((cin, width, width // 2 if i < len(self.dim_mult) - 1 else None))
        return plan


def random_qwen_vae_weights(cfg: QwenVaeConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    w: dict[str, torch.Tensor] = {}

    def conv3(name, o, i, k):
        w[name + ".weight"], w[name + ".bias"] = torch.randn(o, i, k, k, k, generator=g) * std, torch.randn(o, generator=g) * std

    def conv2(name, o, i, k):
        w[name + ".weight"], w[name + ".bias"] = torch.randn(o, i, k, k, generator=g) * std, torch.randn(o, generator=g) * std

    def gamma(name, c, dims=3):
        w[name + ".gamma"] = 1.0 + torch.randn(c, *([1] * dims), generator=g) * 0.1

    def res(p, cin, cout):
        gamma(p + ".norm1", cin)
        conv3(p + ".conv1", cout, cin, 3)
        gamma(p + ".norm2", cout)
        conv3(p + ".conv2", cout, cout, 3)
        if cin != cout:
            conv3(p + ".conv_shortcut", cout, cin, 1)

    top = cfg.base_dim * cfg.dim_mult[-1]
    conv3("post_quant_conv", cfg.z_dim, cfg.z_dim, 1)
    conv3("decoder.conv_in", top, cfg.z_dim, 3)
    res("decoder.mid_block.resnets.0", top, top)
    res("decoder.mid_block.resnets.1", top, top)
    a = "decoder.mid_block.attentions.0"
    gamma(a + ".norm", top, dims=2)
    conv2(a + ".to_qkv", 3 * top, top, 1)
    conv2(a + ".proj", top, top, 1)
    for i, (cin, width, up) in enumerate(cfg.up_plan()):
        for j in range(cfg.num_res_blocks + 1):
            res(f"decoder.up_blocks.{i}.resnets.{j}", cin if j == 0 else width, width)
        if up is not None:
            conv2(f"decoder.up_blocks.{i}.upsamplers.0.resample.1", up, width, 3)
    gamma("decoder.norm_out", cfg.base_dim)
    conv3("decoder.conv_out", 3, cfg.base_dim, 3)
    return w


class QwenVaeDecoder:
    def __init__(self, cfg: QwenVaeConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w: dict[str, torch.Tensor] = {}
        for k, v in weights.items():
            if not k.startswith(("decoder.", "post_quant_conv.")):
                continue
            if k.endswith(".weight") and v.dim() == 5:
                v = v[:, :, -1]                              # the only temporal tap a single frame reaches
            if k.endswith(".gamma"):
                v = v.reshape(1, -1, 1, 1)
            self.w[k] = v.to(device=self.device, dtype=dtype).contiguous()
        self.mean = torch.tensor(LATENTS_MEAN[: cfg.z_dim], device=self.device, dtype=dtype).view(1, -1, 1, 1)
        self.std = torch.tensor(LATENTS_STD[: cfg.z_dim], device=self.device, dtype=dtype).view(1, -1, 1, 1)

    def _conv(self, x, name, pad):
        return F.conv2d(x, self.w[name + ".weight"], self.w[name + ".bias"], padding=pad)

    def _norm(self, x, name):
        xf = x.float()
        c = x.shape[1]
        y = xf / torch.sqrt(xf.pow(2).sum(1, keepdim=True) + NORM_EPS) * (c ** 0.5) * self.w[name + ".gamma"].float()
        return y.to(x.dtype)

    def _res(self, x, p):
        h = self._conv(F.silu(self._norm(x, p + ".norm1")), p + ".conv1", 1)
        h = self._conv(F.silu(self._norm(h, p + ".norm2")), p + ".conv2", 1)
        return h + (self._conv(x, p + ".conv_shortcut", 0) if p + ".conv_shortcut.weight" in self.w else x)

    def _attention(self, x, p):
        B, C, H, W = x.shape
        q, k, v = self._conv(self._norm(x, p + ".norm"), p + ".to_qkv", 0).reshape(B, 3, C, H * W).transpose(2, 3).unbind(1)
        o = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]          # one head of width C
        return x + self._conv(o.transpose(1, 2).reshape(B, C, H, W), p + ".proj", 0)

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """Normalised latents [B, 16, h, w] -> image [B, 3, 8h, 8w] in about [-1, 1]."""
        z = latents.to(self.device, self.dtype) * self.std + self.mean
        h = self._conv(self._conv(z, "post_quant_conv", 0), "decoder.conv_in", 1)
        h = self._res(h, "decoder.mid_block.resnets.0")
        h = self._attention(h, "decoder.mid_block.attentions.0")
        h = self._res(h, "decoder.mid_block.resnets.1")
        for i, (_, _, up) in enumerate(self.cfg.up_plan()):
            for j in range(self.cfg.num_res_blocks + 1):
                h = self._res(h, f"decoder.up_blocks.{i}.resnets.{j}")
            if up is not None:
                h = self._conv(F.interpolate(h, scale_factor=2, mode="nearest"),
                               f"decoder.up_blocks.{i}.upsamplers.0.resample.1", 1)
        return self._conv(F.silu(self._norm(h, "decoder.norm_out")), "decoder.conv_out", 1)


# =================================================================================================================
# the same autoencoder over time (Wan 2.1 video latents)
# =================================================================================================================
def random_wan_vae_weights(cfg: QwenVaeConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """The image checkpoint's tensors plus the temporal-upsampling convolutions of the first two up blocks."""
    w = random_qwen_vae_weights(cfg, seed, std)
    g = torch.Generator().manual_seed(seed + 101)
    for i, (_, width, up) in enumerate(cfg.up_plan()):
        if up is not None and i < 2:
            w[f"decoder.up_blocks.{i}.upsamplers.0.time_conv.weight"] = torch.randn(2 * width, width, 3, 1, 1, generator=g) * std
            w[f"decoder.up_blocks.{i}.upsamplers.0.time_conv.bias"] = torch.randn(2 * width, generator=g) * std
    return w


class WanVaeDecoder:
    """Video decode of the causal 3-D autoencoder (parity: candle-gen-wan/src/vae16.rs): T latent frames become
    1 + 4 (T - 1) frames. Every convolution is causal in time (two frames of zero history in front). The first two up
    blocks double the frame count of everything after the first frame: frame 0 passes through, and a temporal
    convolution over frames 1.. (with zero history, so it never sees frame 0) produces two frames for each of them. The
    middle attention is per frame."""

    def __init__(self, cfg: QwenVaeConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = {}
        for k, v in weights.items():
            if k.startswith(("decoder.", "post_quant_conv.")):
                if k.endswith(".gamma"):
                    v = v.reshape(1, -1, 1, 1, 1)
                elif k.endswith(".weight") and v.dim() == 4:
                    v = v[:, :, None]                              # 2-D convolutions run per frame
                self.w[k] = v.to(device=self.device, dtype=dtype).contiguous()
        self.mean = torch.tensor(LATENTS_MEAN[: cfg.z_dim], device=self.device, dtype=dtype).view(1, -1, 1, 1, 1)
        self.std = torch.tensor(LATENTS_STD[: cfg.z_dim], device=self.device, dtype=dtype).view(1, -1, 1, 1, 1)

    def _conv(self, x, name, pad):
        w = self.w[name + ".weight"]
        kt = w.shape[2]
        return F.conv3d(F.pad(x, (pad, pad, pad, pad, kt - 1, 0)), w, self.w[name + ".bias"])

    def _norm(self, x, name):
        xf = x.float()
        y = xf / torch.sqrt(xf.pow(2).sum(1, keepdim=True) + NORM_EPS) * (x.shape[1] ** 0.5) * self.w[name + ".gamma"].float()
        return y.to(x.dtype)

    def _res(self, x, p):
        h = self._conv(F.silu(self._norm(x, p + ".norm1")), p + ".conv1", 1)
        h = self._conv(F.silu(self._norm(h, p + ".norm2")), p + ".conv2", 1)
        return h + (self._conv(x, p + ".conv_shortcut", 0) if p + ".conv_shortcut.weight" in self.w else x)

    def _attention(self, x, p):
        B, C, T, H, W = x.shape
        qkv = self._conv(self._norm(x, p + ".norm"), p + ".to_qkv", 0)                      # [B, 3C, T, H, W]
        q, k, v = qkv.permute(0, 2, 1, 3, 4).reshape(B * T, 3, C, H * W).transpose(2, 3).unbind(1)
        o = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
        o = o.transpose(1, 2).reshape(B, T, C, H, W).permute(0, 2, 1, 3, 4)
        return x + self._conv(o, p + ".proj", 0)

    def _upsample(self, x, p, temporal: bool):
        B, C, T, H, W = x.shape
        if temporal and T > 1:
            y = self._conv(x[:, :, 1:], p + ".time_conv", 0)                                  # [B, 2C, T - 1, H, W]
            y = torch.stack((y[:, :C], y[:, C:]), 3).reshape(B, C, 2 * (T - 1), H, W)
            x = torch.cat([x[:, :, :1], y], 2)
        T2 = x.shape[2]
        frames = x.permute(0, 2, 1, 3, 4).reshape(B * T2, C, H, W)
        frames = F.interpolate(frames, scale_factor=2, mode="nearest")
        x = frames.reshape(B, T2, C, 2 * H, 2 * W).permute(0, 2, 1, 3, 4)
        return self._conv(x, p + ".resample.1", 1)

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """Normalised latents [B, 16, T, h, w] -> video [B, 3, 1 + 4 (T - 1), 8h, 8w] in about [-1, 1]."""
        z = latents.to(self.device, self.dtype) * self.std + self.mean
        h = self._conv(self._conv(z, "post_quant_conv", 0), "decoder.conv_in", 1)
        h = self._res(h, "decoder.mid_block.resnets.0")
        h = self._attention(h, "decoder.mid_block.attentions.0")
        h = self._res(h, "decoder.mid_block.resnets.1")
        for i, (_, _, up) in enumerate(self.cfg.up_plan()):
            for j in range(self.cfg.num_res_blocks + 1):
                h = self._res(h, f"decoder.up_blocks.{i}.resnets.{j}")
            if up is not None:
                h = self._upsample(h, f"decoder.up_blocks.{i}.upsamplers.0", temporal=i < 2)
        return self._conv(F.silu(self._norm(h, "decoder.norm_out")), "decoder.conv_out", 1)


def random_wan_vae_encoder_weights(cfg: QwenVaeConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """Encoder + quant_conv tensors of the video autoencoder (diffusers spelling)."""
    g = torch.Generator().manual_seed(seed + 211)
    rn = lambda *s: torch.randn(*s, generator=g)      # noqa: E731
    w: dict[str, torch.Tensor] = {}

    def conv3(name, o, i, k):
        w[name + ".weight"], w[name + ".bias"] = rn(o, i, k, k, k) * std, rn(o) * std

    def res(p, cin, cout):
        w[p + ".norm1.gamma"], w[p + ".norm2.gamma"] = 1.0 + rn(cin, 1, 1, 1) * 0.05, 1.0 + rn(cout, 1, 1, 1) * 0.05
        conv3(p + ".conv1", cout, cin, 3)
        conv3(p + ".conv2", cout, cout, 3)
        if cin != cout:
            conv3(p + ".conv_shortcut", cout, cin, 1)

    b = cfg.base_dim
    dims = [b * m for m in cfg.dim_mult]
    conv3("encoder.conv_in", b, 3, 3)
    idx, cin = 0, b
    for s, d in enumerate(dims):
        for j in range(cfg.num_res_blocks):
            res(f"encoder.down_blocks.{idx}", cin if j == 0 else d, d)
            idx += 1
        cin = d
        if s < len(dims) - 1:
            p = f"encoder.down_blocks.{idx}"
            w[p + ".resample.1.weight"], w[p + ".resample.1.bias"] = rn(d, d, 3, 3) * std, rn(d) * std
            if s > 0:
                w[p + ".time_conv.weight"], w[p + ".time_conv.bias"] = rn(d, d, 3, 1, 1) * std, rn(d) * std
            idx += 1
    top = dims[-1]
    res("encoder.mid_block.resnets.0", top, top)
    res("encoder.mid_block.resnets.1", top, top)
    a = "encoder.mid_block.attentions.0"
    w[a + ".norm.gamma"] = 1.0 + rn(top, 1, 1) * 0.05
    w[a + ".to_qkv.weight"], w[a + ".to_qkv.bias"] = rn(3 * top, top, 1, 1) * std, rn(3 * top) * std
    w[a + ".proj.weight"], w[a + ".proj.bias"] = rn(top, top, 1, 1) * std, rn(top) * std
    w["encoder.norm_out.gamma"] = 1.0 + rn(top, 1, 1, 1) * 0.05
    conv3("encoder.conv_out", 2 * cfg.z_dim, top, 3)
    conv3("quant_conv", 2 * cfg.z_dim, 2 * cfg.z_dim, 1)
    return w


class WanVaeEncoder(WanVaeDecoder):
    """Video encode of the causal 3-D autoencoder (parity: candle-gen-wan/src/vae16.rs:74-300,554-598): 1 + 4n frames
    become 1 + n normalised latent frames (the posterior mean). Stages 1 and 2 halve the frame count of everything
    after the first frame: frame 0 passes through untouched and a stride-2 three-tap temporal convolution runs over
    the whole clip (the reference streams it in chunks of 1, 4, 4, ... frames with one cached frame, which is the same
    convolution). Spatial downsampling is a stride-2 3x3 convolution padded by one row / column at the bottom / right."""

    def __init__(self, cfg: QwenVaeConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = {}
        for k, v in weights.items():
            if k.startswith(("encoder.", "quant_conv.")):
                if k.endswith(".gamma"):
                    v = v.reshape(1, -1, 1, 1, 1)
                elif k.endswith(".weight") and v.dim() == 4:
                    v = v[:, :, None]
                self.w[k] = v.to(device=self.device, dtype=dtype).contiguous()
        self.mean = torch.tensor(LATENTS_MEAN[: cfg.z_dim], device=self.device, dtype=torch.float32).view(1, -1, 1, 1, 1)
        self.std = torch.tensor(LATENTS_STD[: cfg.z_dim], device=self.device, dtype=torch.float32).view(1, -1, 1, 1, 1)

    @torch.no_grad()
    def encode(self, video: torch.Tensor) -> torch.Tensor:
        """[B, 3, 1 + 4n, H, W] in [-1, 1] -> normalised latents [B, 16, 1 + n, H / 8, W / 8] (fp32)."""
        T = video.shape[2]
        if (T - 1) % 4:
            raise ValueError(f"the causal encoder consumes 1 + 4n frames (got {T})")
        cfg = self.cfg
        h = self._conv(video.to(self.device, self.dtype), "encoder.conv_in", 1)
        idx, stages = 0, len(cfg.dim_mult)
        for s in range(stages):
            for _ in range(cfg.num_res_blocks):
                h = self._res(h, f"encoder.down_blocks.{idx}")
                idx += 1
            if s < stages - 1:
                p = f"encoder.down_blocks.{idx}"
                h = F.conv3d(F.pad(h, (0, 1, 0, 1)), self.w[p + ".resample.1.weight"], self.w[p + ".resample.1.bias"],
                             stride=(1, 2, 2))
                if p + ".time_conv.weight" in self.w and h.shape[2] > 1:
                    rest = F.conv3d(h, self.w[p + ".time_conv.weight"], self.w[p + ".time_conv.bias"], stride=(2, 1, 1))
                    h = torch.cat([h[:, :, :1], rest], dim=2)
                idx += 1
        h = self._res(h, "encoder.mid_block.resnets.0")
        h = self._attention(h, "encoder.mid_block.attentions.0")
        h = self._res(h, "encoder.mid_block.resnets.1")
        h = self._conv(F.silu(self._norm(h, "encoder.norm_out")), "encoder.conv_out", 1)
        mu = self._conv(h, "quant_conv", 0)[:, : cfg.z_dim].float()
        return (mu - self.mean) / self.std


# ---- Wan2.2 z48 residual autoencoder (decode side) -----------------------------------------------------------------------
LATENTS48_MEAN = (-0.2289, -0.0052, -0.1323, -0.2339, -0.2799, 0.0174, 0.1838, 0.1557, -0.1382, 0.0542, 0.2813, 0.0891, 0.157,
                  -0.0098, 0.0375, -0.1825, -0.2246, -0.1207, -0.0698, 0.5109, 0.2665, -0.2108, -0.2158, 0.2502, -0.2055, -0.0322,
                  0.1109, 0.1567, -0.0729, 0.0899, -0.2799, -0.123, -0.0313, -0.1649, 0.0117, 0.0723, -0.2839, -0.2083, -0.052,
                  0.3748, 0.0152, 0.1957, 0.1433, -0.2944, 0.3573, -0.0548, -0.1681, -0.0667)
LATENTS48_STD = (0.4765, 1.0364, 0.4514, 1.1677, 0.5313, 0.499, 0.4818, 0.5013, 0.8158, 1.0344, 0.5894, 1.0901, 0.6885, 0.6165,
                 0.8454, 0.4978, 0.5759, 0.3523, 0.7135, 0.6804, 0.5833, 1.4146, 0.8986, 0.5659, 0.7069, 0.5338, 0.4889, 0.4917,
                 0.4069, 0.4999, 0.6866, 0.4093, 0.5709, 0.6065, 0.6415, 0.4944, 0.5726, 1.2042, 0.5458, 1.6887, 0.3971, 1.06,
                 0.3943, 0.5537, 0.5444, 0.4089, 0.7468, 0.7744)


@dataclass
class Wan22VaeConfig:
    z_dim: int = 48
    base_dim: int = 256
    num_res_blocks: int = 2
    patch_size: int = 2
    out_channels: int = 3

    @property
    def dims(self) -> tuple[int, ...]:
        b = self.base_dim
        return (4 * b, 4 * b, 4 * b, 2 * b, b)


class Wan22VaeDecoder(WanVaeDecoder):
    """Decode side of the Wan2.2 residual autoencoder (parity: candle-gen-wan/src/vae.rs): latents [B, 48, T, h, w] ->
    video [B, 3, 1 + 4 (T - 1), 16 h, 16 w]. Four up blocks of three residual units; the first two double time and
    space, the third space only, and each of those three adds a parameter-free shortcut: the block input with its
    channels repeated and folded into the (time, row, column) factors (the leading frame of a time-doubling fold is
    dropped, matching the first-frame rule of the learned path). The output convolution emits 12 channels that unfold
    2 x 2 into RGB."""

    def __init__(self, cfg: Wan22VaeConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = {}
        for k, v in weights.items():
            if k.startswith(("decoder.", "post_quant_conv.")):
                if k.endswith(".gamma"):
                    v = v.reshape(1, -1, 1, 1, 1)
                elif k.endswith(".weight") and v.dim() == 4:
                    v = v[:, :, None]
                self.w[k] = v.to(device=self.device, dtype=dtype).contiguous()
        n = cfg.z_dim
        self.mean = torch.tensor((LATENTS48_MEAN * (n // 48 + 1))[:n], device=self.device, dtype=dtype).view(1, -1, 1, 1, 1)
        self.std = torch.tensor((LATENTS48_STD * (n // 48 + 1))[:n], device=self.device, dtype=dtype).view(1, -1, 1, 1, 1)

    @staticmethod
    def dup_shortcut(x: torch.Tensor, out_c: int, ft: int, fs: int) -> torch.Tensor:
        B, C, T, H, W = x.shape
        rep = out_c * ft * fs * fs // C
        y = x[:, :, None].expand(B, C, rep, T, H, W).reshape(B, out_c, ft, fs, fs, T, H, W)
        y = y.permute(0, 1, 5, 2, 6, 3, 7, 4).reshape(B, out_c, T * ft, H * fs, W * fs)
        return y[:, :, ft - 1:] if ft > 1 else y

    def _up(self, x, p, temporal: bool):
        B, C, T, H, W = x.shape
        if temporal:
            if T > 1:
                y = self._conv(x[:, :, 1:], p + ".time_conv", 0)
                y = torch.stack((y[:, :C], y[:, C:]), 3).reshape(B, C, 2 * (T - 1), H, W)
                x = torch.cat([x[:, :, :1], y], 2)
            else:
                x = x[:, :, :1]
        T2 = x.shape[2]
        fr = F.interpolate(x.permute(0, 2, 1, 3, 4).reshape(B * T2, C, H, W), scale_factor=2, mode="nearest")
        return self._conv(fr.reshape(B, T2, C, 2 * H, 2 * W).permute(0, 2, 1, 3, 4), p + ".resample.1", 1)

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        cfg, dims = self.cfg, self.cfg.dims
        z = latents.to(self.device, self.dtype) * self.std + self.mean
        h = self._conv(self._conv(z, "post_quant_conv", 0), "decoder.conv_in", 1)
        h = self._res(h, "decoder.mid_block.resnets.0")
        h = self._attention(h, "decoder.mid_block.attentions.0")
        h = self._res(h, "decoder.mid_block.resnets.1")
        for i in range(4):
            x0 = h
            for j in range(cfg.num_res_blocks + 1):
                h = self._res(h, f"decoder.up_blocks.{i}.resnets.{j}")
            if i != 3:
                h = self._up(h, f"decoder.up_blocks.{i}.upsampler", temporal=i < 2)
                h = h + self.dup_shortcut(x0, dims[i + 1], 2 if i < 2 else 1, 2)
        h = self._conv(F.silu(self._norm(h, "decoder.norm_out")), "decoder.conv_out", 1)       # [B, 3 p p, T', 8h, 8w]
        B, _, T, H, W = h.shape
        p, c = cfg.patch_size, cfg.out_channels
        return h.reshape(B, c, p, p, T, H, W).permute(0, 1, 4, 5, 3, 6, 2).reshape(B, c, T, H * p, W * p)


def random_wan22_vae_weights(cfg: Wan22VaeConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    w: dict[str, torch.Tensor] = {}

    def conv3(name, o, i, k):
        w[name + ".weight"] = torch.randn(o, i, *k, generator=g) * std
        w[name + ".bias"] = torch.randn(o, generator=g) * 0.01

    def gamma(name, c, dims=3):
        w[name + ".gamma"] = 1 + torch.randn(c, *([1] * dims), generator=g) * 0.05

    def res(p, cin, cout):
        gamma(p + ".norm1", cin)
        conv3(p + ".conv1", cout, cin, (3, 3, 3))
        gamma(p + ".norm2", cout)
        conv3(p + ".conv2", cout, cout, (3, 3, 3))
        if cin != cout:
            conv3(p + ".conv_shortcut", cout, cin, (1, 1, 1))

    d = cfg.dims
    conv3("post_quant_conv", cfg.z_dim, cfg.z_dim, (1, 1, 1))
    conv3("decoder.conv_in", d[0], cfg.z_dim, (3, 3, 3))
    res("decoder.mid_block.resnets.0", d[0], d[0])
    res("decoder.mid_block.resnets.1", d[0], d[0])
    a = "decoder.mid_block.attentions.0"
    gamma(a + ".norm", d[0], 2)
    w[a + ".to_qkv.weight"], w[a + ".to_qkv.bias"] = torch.randn(3 * d[0], d[0], 1, 1, generator=g) * std, torch.zeros(3 * d[0])
    w[a + ".proj.weight"], w[a + ".proj.bias"] = torch.randn(d[0], d[0], 1, 1, generator=g) * std, torch.zeros(d[0])
    for i in range(4):
        cur = d[i]
        for j in range(cfg.num_res_blocks + 1):
            res(f"decoder.up_blocks.{i}.resnets.{j}", cur, d[i + 1])
            cur = d[i + 1]
        if i != 3:
            u = f"decoder.up_blocks.{i}.upsampler"
            if i < 2:
                conv3(u + ".time_conv", 2 * cur, cur, (3, 1, 1))
            w[u + ".resample.1.weight"], w[u + ".resample.1.bias"] = torch.randn(cur, cur, 3, 3, generator=g) * std, torch.zeros(cur)
    gamma("decoder.norm_out", d[4])
    conv3("decoder.conv_out", cfg.out_channels * cfg.patch_size ** 2, d[4], (3, 3, 3))
    return w
