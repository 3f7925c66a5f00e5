"""FLUX AutoEncoder decoder (16-channel latents -> RGB): fp32 oracle and the sm_100a channels-last model.

Structure (parity: candle-gen-flux/src/vae/native.rs:80-399): conv_in -> mid (ResnetBlock, single-head AttnBlock,
ResnetBlock) -> 4 up levels (ch_mult [1, 2, 4, 4] reversed, num_res_blocks + 1 ResnetBlocks each, nearest 2x
upsample + conv3x3 between levels) -> GroupNorm(32) -> swish -> conv_out. Latents are unscaled first:
z / scale_factor + shift_factor.

GPU execution keeps activations NHWC bf16: every convolution is a tcgen05 GEMM (3x3 through a patch gather, 1x1
directly) with bias and the residual add fused in the epilogue; GroupNorm + SiLU is one fused pass after a
statistics pass; the mid-block attention is GEMM -> row softmax -> GEMM."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops


@dataclass
class VaeConfig:
    ch: int = 128
    out_ch: int = 3
    ch_mult: tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    z_channels: int = 16
    scale_factor: float = 0.3611
    shift_factor: float = 0.1159

    @staticmethod
    def tiny() -> "VaeConfig":
        return VaeConfig(ch=32, ch_mult=(1, 2), num_res_blocks=1, z_channels=16)


def random_vae_weights(cfg: VaeConfig, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"):
    g = torch.Generator(device=device).manual_seed(seed)
    w: dict[str, torch.Tensor] = {}

    def conv(name, cout, cin, k):
        w[name + ".weight"] = (torch.randn(cout, cin, k, k, generator=g, device=device) * std / (k * (cin ** 0.5) / 4)
                               ).to(dtype)
        w[name + ".bias"] = (torch.randn(cout, generator=g, device=device) * 0.01).to(dtype)

    def norm(name, c):
        w[name + ".weight"] = (1 + 0.1 * torch.randn(c, generator=g, device=device)).to(dtype)
        w[name + ".bias"] = (0.05 * torch.randn(c, generator=g, device=device)).to(dtype)

    def res(name, cin, cout):
        norm(name + ".norm1", cin)
        conv(name + ".conv1", cout, cin, 3)
        norm(name + ".norm2", cout)
        conv(name + ".conv2", cout, cout, 3)
        if cin != cout:
            conv(name + ".nin_shortcut", cout, cin, 1)

    block_in = cfg.ch * cfg.ch_mult[-1]
    conv("decoder.conv_in", block_in, cfg.z_channels, 3)
    res("decoder.mid.block_1", block_in, block_in)
    norm("decoder.mid.attn_1.norm", block_in)
    for n in ("q", "k", "v", "proj_out"):
        conv(f"decoder.mid.attn_1.{n}", block_in, block_in, 1)
    res("decoder.mid.block_2", block_in, block_in)
    for lvl in reversed(range(len(cfg.ch_mult))):
        block_out = cfg.ch * cfg.ch_mult[lvl]
        for i in range(cfg.num_res_blocks + 1):
            res(f"decoder.up.{lvl}.block.{i}", block_in, block_out)
            block_in = block_out
        if lvl != 0:
            conv(f"decoder.up.{lvl}.upsample.conv", block_in, block_in, 3)
    norm("decoder.norm_out", block_in)
    conv("decoder.conv_out", cfg.out_ch, block_in, 3)
    return w


class OracleVaeDecoder:
    def __init__(self, cfg: VaeConfig, weights, dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}

    def _conv(self, x, name, pad):
        return F.conv2d(x, self.w[name + ".weight"], self.w[name + ".bias"], padding=pad)

    def _gn(self, x, name, silu):
        y = F.group_norm(x, 32, self.w[name + ".weight"], self.w[name + ".bias"], 1e-6)
        return F.silu(y) if silu else y

    def _res(self, x, name):
        h = self._conv(self._gn(x, name + ".norm1", True), name + ".conv1", 1)
        h = self._conv(self._gn(h, name + ".norm2", True), name + ".conv2", 1)
        if (name + ".nin_shortcut.weight") in self.w:
            x = self._conv(x, name + ".nin_shortcut", 0)
        return x + h

    def _attn(self, x, name):
        h = self._gn(x, name + ".norm", False)
        q, k, v = (self._conv(h, f"{name}.{n}", 0) for n in "qkv")
        B, C, H, W = q.shape
        q, k, v = (t.flatten(2).transpose(1, 2) for t in (q, k, v))
        o = torch.softmax(q @ k.transpose(1, 2) * C ** -0.5, -1) @ v
        return x + self._conv(o.transpose(1, 2).reshape(B, C, H, W), name + ".proj_out", 0)

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """z [B, 16, h, w] (scaled latents) -> image [B, 3, 8h.., 8w..] in roughly [-1, 1]."""
        cfg = self.cfg
        h = self._conv(z / cfg.scale_factor + cfg.shift_factor, "decoder.conv_in", 1)
        h = self._res(h, "decoder.mid.block_1")
        h = self._attn(h, "decoder.mid.attn_1")
        h = self._res(h, "decoder.mid.block_2")
        for lvl in reversed(range(len(cfg.ch_mult))):
            for i in range(cfg.num_res_blocks + 1):
                h = self._res(h, f"decoder.up.{lvl}.block.{i}")
            if lvl != 0:
                h = self._conv(F.interpolate(h, scale_factor=2, mode="nearest"), f"decoder.up.{lvl}.upsample.conv", 1)
        return self._conv(self._gn(h, "decoder.norm_out", True), "decoder.conv_out", 1)


def random_vae_encoder_weights(cfg: VaeConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """Random encoder tensors under the `encoder.*` names of the latent-diffusion layout."""
    g = torch.Generator().manual_seed(seed)
    w: dict[str, torch.Tensor] = {}

    def conv(name, cout, cin, k):
        w[name + ".weight"] = torch.randn(cout, cin, k, k, generator=g) * std / (k * (cin ** 0.5) / 4)
        w[name + ".bias"] = torch.randn(cout, generator=g) * 0.01

    def norm(name, c):
        w[name + ".weight"], w[name + ".bias"] = 1 + 0.1 * torch.randn(c, generator=g), 0.05 * torch.randn(c, generator=g)

    def res(name, cin, cout):
        norm(name + ".norm1", cin)
        conv(name + ".conv1", cout, cin, 3)
        norm(name + ".norm2", cout)
        conv(name + ".conv2", cout, cout, 3)
        if cin != cout:
            conv(name + ".nin_shortcut", cout, cin, 1)

    conv("encoder.conv_in", cfg.ch, 3, 3)
    block_in = cfg.ch
    for lvl, m in enumerate(cfg.ch_mult):
        for i in range(cfg.num_res_blocks):
            res(f"encoder.down.{lvl}.block.{i}", block_in, cfg.ch * m)
            block_in = cfg.ch * m
        if lvl != len(cfg.ch_mult) - 1:
            conv(f"encoder.down.{lvl}.downsample.conv", block_in, block_in, 3)
    res("encoder.mid.block_1", block_in, block_in)
    norm("encoder.mid.attn_1.norm", block_in)
    for n in ("q", "k", "v", "proj_out"):
        conv(f"encoder.mid.attn_1.{n}", block_in, block_in, 1)
    res("encoder.mid.block_2", block_in, block_in)
    norm("encoder.norm_out", block_in)
    conv("encoder.conv_out", 2 * cfg.z_channels, block_in, 3)
    return w


class OracleVaeEncoder(OracleVaeDecoder):
    """Image -> latent mean (the deterministic encode used for reference-guided generation and for caching training
    latents): strided convolutions with (0, 1, 0, 1) padding between levels, the same residual / attention blocks as the
    decoder, the first half of `conv_out`'s channels is the mean; the stored latent is (mean - shift) * scale."""

    @torch.no_grad()
    def encode(self, image: torch.Tensor) -> torch.Tensor:
        """image [B, 3, H, W] in [-1, 1] -> scaled latents [B, z, H/8.., W/8..]."""
        cfg = self.cfg
        dev = next(iter(self.w.values()))
        h = self._conv(image.to(dev.device, dev.dtype), "encoder.conv_in", 1)
        for lvl in range(len(cfg.ch_mult)):
            for i in range(cfg.num_res_blocks):
                h = self._res(h, f"encoder.down.{lvl}.block.{i}")
            if lvl != len(cfg.ch_mult) - 1:
                n = f"encoder.down.{lvl}.downsample.conv"
                h = F.conv2d(F.pad(h, (0, 1, 0, 1)), self.w[n + ".weight"], self.w[n + ".bias"], stride=2)
        h = self._res(h, "encoder.mid.block_1")
        h = self._attn(h, "encoder.mid.attn_1")
        h = self._res(h, "encoder.mid.block_2")
        moments = self._conv(self._gn(h, "encoder.norm_out", True), "encoder.conv_out", 1)
        if "quant_conv.weight" in self.w:               # SDXL-style autoencoders: a 1x1 convolution over the moments
            moments = self._conv(moments, "quant_conv", 0)
        return (moments[:, : cfg.z_channels] - cfg.shift_factor) * cfg.scale_factor


class VaeDecoderGpu:
    def __init__(self, cfg: VaeConfig, device: torch.device | None = None):
        self.cfg = cfg
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.w: dict[str, torch.Tensor] = {}
        self.launches = 0

    def load_state_dict(self, weights) -> "VaeDecoderGpu":
        self.w = {}
        for k, v in weights.items():
            if not k.startswith("decoder."):          # full autoencoder checkpoints also carry the encoder
                continue
            t = v.to(device=self.device, dtype=torch.float32)
            if t.dim() == 4:   # OIHW -> [O, (kh, kw, I)] matching the patch-gather column order
                o, i, kh, kw = t.shape
                t = t.permute(0, 2, 3, 1).reshape(o, kh * kw * i)
                if t.shape[1] % 8:
                    raise ValueError(f"{k}: reduction size {t.shape[1]} is not a multiple of 8")
                if o % 8:      # pad tiny output widths (conv_out -> RGB) so rows stay 16-byte aligned
                    t = torch.cat([t, torch.zeros(8 - o % 8, t.shape[1], device=t.device)], 0)
            elif k.endswith("conv_out.bias") and t.numel() % 8:
                t = torch.cat([t, torch.zeros(8 - t.numel() % 8, device=t.device)])
            self.w[k] = t.bfloat16().contiguous()
        return self

    def init_random(self, seed: int = 0) -> "VaeDecoderGpu":
        return self.load_state_dict(random_vae_weights(self.cfg, seed, device=self.device))

    def _conv3(self, x, name, residual=None):
        self.launches += 1 if ops.conv3x3_supported(x) else 2
        return ops.conv3x3_nhwc(x, self.w[name + ".weight"], self.w[name + ".bias"], residual)

    def _conv1(self, x, name, residual=None):
        N, H, W, C = x.shape
        res = residual.reshape(N * H * W, -1) if residual is not None else None
        y = ops.gemm_bf16(x.reshape(N * H * W, C), self.w[name + ".weight"], bias=self.w[name + ".bias"], residual=res)
        self.launches += 1
        return y.view(N, H, W, -1)

    def _gn(self, x, name, silu):
        self.launches += 2
        return ops.groupnorm_nhwc(x, self.w[name + ".weight"], self.w[name + ".bias"], 32, 1e-6, silu)

    def _res(self, x, name):
        h = self._conv3(self._gn(x, name + ".norm1", True), name + ".conv1")
        skip = self._conv1(x, name + ".nin_shortcut") if (name + ".nin_shortcut.weight") in self.w else x
        return self._conv3(self._gn(h, name + ".norm2", True), name + ".conv2", residual=skip)

    def _attn(self, x, name):
        N, H, W, C = x.shape
        h = self._gn(x, name + ".norm", False)
        q, k, v = (self._conv1(h, f"{name}.{n}").view(N, H * W, C) for n in "qkv")
        outs = []
        for b in range(N):
            T = H * W
            o = torch.empty((T, C), dtype=torch.bfloat16, device=x.device)
            vt = v[b].t().contiguous()                   # [C, T]: the GEMM wants the reduction dim contiguous
            step = max(128, min(T, (256 << 20) // (T * 4)))
            for lo in range(0, T, step):
                hi = min(T, lo + step)
                s = ops.gemm_bf16(q[b, lo:hi], k[b], out_dtype=torch.float32)      # [rows, T]
                p = ops.softmax_rows(s, C ** -0.5)
                ops.gemm_bf16(p, vt, out=o[lo:hi])
                self.launches += 3
            outs.append(o)
        o = torch.stack(outs).view(N, H, W, C)
        return self._conv1(o, name + ".proj_out", residual=x)

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """z [B, 16, h, w] -> image NHWC bf16 [B, H, W, 8] (channels 0..2 are RGB in roughly [-1, 1])."""
        cfg = self.cfg
        self.launches = 0
        x = (z.float() / cfg.scale_factor + cfg.shift_factor).permute(0, 2, 3, 1).contiguous().bfloat16()
        h = self._conv3(x, "decoder.conv_in")
        h = self._res(h, "decoder.mid.block_1")
        h = self._attn(h, "decoder.mid.attn_1")
        h = self._res(h, "decoder.mid.block_2")
        for lvl in reversed(range(len(cfg.ch_mult))):
            for i in range(cfg.num_res_blocks + 1):
                h = self._res(h, f"decoder.up.{lvl}.block.{i}")
            if lvl != 0:
                h = self._conv3(ops.upsample2x_nhwc(h), f"decoder.up.{lvl}.upsample.conv")
                self.launches += 1
        return self._conv3(self._gn(h, "decoder.norm_out", True), "decoder.conv_out")

    def decode_rgb8(self, z: torch.Tensor) -> torch.Tensor:
        return ops.rgb8_nhwc(self.decode(z))
