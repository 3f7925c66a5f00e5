"""SDXL UNet (parity: candle-gen-sdxl/src/unet/*; checkpoint keys are the diffusers `UNet2DConditionModel` names).

Three resolution levels (320 / 640 / 1280 channels, two residual blocks each on the way down, three on the way up);
the two lower-resolution levels and the middle carry transformer stacks (2 and 10 blocks; self-attention,
cross-attention on the [77, 2048] text context, GEGLU feed-forward; head width 64). The time embedding is the sum of
the timestep embedding and an embedding of (pooled text vector, six size / crop numbers).

One implementation serves both backends: fp32 on the CPU oracle backend; bf16 on a CUDA device, where linear
projections go through the tcgen05 GEMM (`text_encoders.linear`), attention through the tcgen05 attention kernel with
the 64-wide heads zero-padded to its 128, and convolutions and group norms through the framework's library calls."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .nn_dual import adapter_residual

from .dit_flux import timestep_embedding
from .text_encoders import linear


def _narrow_on_kernel() -> bool:
    from ..ops.attention import narrow_heads_on_kernel

    return narrow_heads_on_kernel()


@dataclass
class SdxlUnetConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_out_channels: tuple[int, ...] = (320, 640, 1280)
    layers_per_block: int = 2
    transformer_layers_per_block: tuple[int, ...] = (0, 2, 10)          # 0 = a level without attention
    attention_head_dim: int = 64
    cross_attention_dim: int = 2048
    addition_time_embed_dim: int = 256
    projection_class_embeddings_input_dim: int = 2816
    norm_groups: int = 32
    encoder_hid_dim: int = 0          # Kolors: the text states are 4096 wide and projected to cross_attention_dim first

    @property
    def time_dim(self) -> int:
        return 4 * self.block_out_channels[0]

    @staticmethod
    def from_json(j: dict) -> "SdxlUnetConfig":
        boc = tuple(j.get("block_out_channels", (320, 640, 1280)))
        kinds = j.get("down_block_types", ["DownBlock2D"] + ["CrossAttnDownBlock2D"] * (len(boc) - 1))
        tl = j.get("transformer_layers_per_block", 1)
        tl = [tl] * len(boc) if isinstance(tl, int) else list(tl)
        tl = tuple(n if "CrossAttn" in k else 0 for n, k in zip(tl, kinds))
        heads = j.get("attention_head_dim", [5, 10, 20])              # diffusers stores the head COUNT under this name
        heads = [heads] * len(boc) if isinstance(heads, int) else list(heads)
        return SdxlUnetConfig(in_channels=j.get("in_channels", 4), out_channels=j.get("out_channels", 4),
                              block_out_channels=boc, layers_per_block=j.get("layers_per_block", 2),
                              transformer_layers_per_block=tl, attention_head_dim=boc[-1] // heads[-1],
                              cross_attention_dim=j.get("cross_attention_dim", 2048),
                              addition_time_embed_dim=j.get("addition_time_embed_dim", 256),
                              projection_class_embeddings_input_dim=j.get("projection_class_embeddings_input_dim", 2816),
                              norm_groups=j.get("norm_num_groups", 32), encoder_hid_dim=int(j.get("encoder_hid_dim") or 0))


def unet_plan(cfg: SdxlUnetConfig):
    """The block list both the weight generator and the forward pass walk.
    down: (level, [(resnet in, out)], transformer depth, has downsampler); up: (level, [(in, out)], depth, has upsampler)."""
    boc = cfg.block_out_channels
    down, skips = [], [boc[0]]
    prev = boc[0]
    for lvl, ch in enumerate(boc):
        res = []
        for j in range(cfg.layers_per_block):
            res.append((prev if j == 0 else ch, ch))
            skips.append(ch)
        last = lvl == len(boc) - 1
        if not last:
            skips.append(ch)
        down.append((lvl, res, cfg.transformer_layers_per_block[lvl], not last))
        prev = ch
    up = []
    for i, lvl in enumerate(reversed(range(len(boc)))):
        ch = boc[lvl]
        res = []
        for j in range(cfg.layers_per_block + 1):
            res.append((prev + skips.pop(), ch))
            prev = ch
        up.append((lvl, res, cfg.transformer_layers_per_block[lvl], i < len(boc) - 1))
    return down, up


def random_sdxl_unet_weights(cfg: SdxlUnetConfig, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"
                             ) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device)      # noqa: E731
    w: dict[str, torch.Tensor] = {}
    T = cfg.time_dim

    def lin(name, o, i, bias=True):
        w[name + ".weight"] = (rn(o, i) * std).to(dtype)
        if bias:
            w[name + ".bias"] = (rn(o) * std).to(dtype)

    def conv(name, o, i, k):
        w[name + ".weight"], w[name + ".bias"] = (rn(o, i, k, k) * std).to(dtype), (rn(o) * std).to(dtype)

    def norm(name, c):
        w[name + ".weight"], w[name + ".bias"] = (1.0 + rn(c) * 0.1).to(dtype), (rn(c) * 0.1).to(dtype)

    def resnet(p, cin, cout):
        norm(p + ".norm1", cin)
        conv(p + ".conv1", cout, cin, 3)
        lin(p + ".time_emb_proj", cout, T)
        norm(p + ".norm2", cout)
        conv(p + ".conv2", cout, cout, 3)
        if cin != cout:
            conv(p + ".conv_shortcut", cout, cin, 1)

    def transformer(p, ch, depth):
        norm(p + ".norm", ch)
        lin(p + ".proj_in", ch, ch)
        for k in range(depth):
            b = f"{p}.transformer_blocks.{k}"
            for n in ("norm1", "norm2", "norm3"):
                norm(f"{b}.{n}", ch)
            for a, kv in (("attn1", ch), ("attn2", cfg.cross_attention_dim)):
                lin(f"{b}.{a}.to_q", ch, ch, bias=False)
                lin(f"{b}.{a}.to_k", ch, kv, bias=False)
                lin(f"{b}.{a}.to_v", ch, kv, bias=False)
                lin(f"{b}.{a}.to_out.0", ch, ch)
            lin(f"{b}.ff.net.0.proj", 8 * ch, ch)
            lin(f"{b}.ff.net.2", ch, 4 * ch)
        lin(p + ".proj_out", ch, ch)

    down, up = unet_plan(cfg)
    conv("conv_in", cfg.block_out_channels[0], cfg.in_channels, 3)
    lin("time_embedding.linear_1", T, cfg.block_out_channels[0])
    lin("time_embedding.linear_2", T, T)
    lin("add_embedding.linear_1", T, cfg.projection_class_embeddings_input_dim)
    lin("add_embedding.linear_2", T, T)
    if cfg.encoder_hid_dim:
        lin("encoder_hid_proj", cfg.cross_attention_dim, cfg.encoder_hid_dim)
    for lvl, res, depth, sampler in down:
        for j, (cin, cout) in enumerate(res):
            resnet(f"down_blocks.{lvl}.resnets.{j}", cin, cout)
            if depth:
                transformer(f"down_blocks.{lvl}.attentions.{j}", cout, depth)
        if sampler:
            conv(f"down_blocks.{lvl}.downsamplers.0.conv", res[-1][1], res[-1][1], 3)
    top = cfg.block_out_channels[-1]
    resnet("mid_block.resnets.0", top, top)
    transformer("mid_block.attentions.0", top, cfg.transformer_layers_per_block[-1])
    resnet("mid_block.resnets.1", top, top)
    for i, (lvl, res, depth, sampler) in enumerate(up):
        for j, (cin, cout) in enumerate(res):
            resnet(f"up_blocks.{i}.resnets.{j}", cin, cout)
            if depth:
                transformer(f"up_blocks.{i}.attentions.{j}", cout, depth)
        if sampler:
            conv(f"up_blocks.{i}.upsamplers.0.conv", res[-1][1], res[-1][1], 3)
    norm("conv_norm_out", cfg.block_out_channels[0])
    conv("conv_out", cfg.out_channels, cfg.block_out_channels[0], 3)
    return w


class SdxlUnet:
    def __init__(self, cfg: SdxlUnetConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = {k: v.to(device=self.device, dtype=dtype).contiguous() for k, v in weights.items()}
        self.plan = unet_plan(cfg)
        self.lora = None

    def _lin(self, x, name):
        y = linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))
        if self.lora is not None and name in self.lora:
            y = y + adapter_residual(self.lora[name], x)
        return y

    def _conv(self, x, name, stride=1, pad=1):
        return F.conv2d(x, self.w[name + ".weight"], self.w[name + ".bias"], stride=stride, padding=pad)

    def _gn(self, x, name, eps, silu=False):
        y = F.group_norm(x.float(), self.cfg.norm_groups, self.w[name + ".weight"].float(), self.w[name + ".bias"].float(), eps)
        return (F.silu(y) if silu else y).to(x.dtype)

    def _ln(self, x, name):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(),
                            1e-5).to(x.dtype)

    def _resnet(self, x, p, emb_act):
        h = self._conv(self._gn(x, p + ".norm1", 1e-5, silu=True), p + ".conv1")
        h = h + self._lin(emb_act, p + ".time_emb_proj")[:, :, None, None]
        h = self._conv(self._gn(h, p + ".norm2", 1e-5, silu=True), p + ".conv2")
        return h + (self._conv(x, p + ".conv_shortcut", pad=0) if p + ".conv_shortcut.weight" in self.w else x)

    def _attention(self, x, ctx, p):
        B, S, C = x.shape
        nh = C // self.cfg.attention_head_dim
        q = self._lin(x, p + ".to_q").view(B, S, nh, -1)
        k = self._lin(ctx, p + ".to_k").view(B, ctx.shape[1], nh, -1)
        v = self._lin(ctx, p + ".to_v").view(B, ctx.shape[1], nh, -1)
        hd = q.shape[-1]
        if q.is_cuda and q.dtype == torch.bfloat16 and hd <= 128 and hd % 8 == 0 and _narrow_on_kernel():
            from .. import ops

            o = ops.dense_attention_padded(q, k, v, scale=hd ** -0.5)          # tcgen05 kernel, heads zero-padded to 128
        else:
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, S, C)
        return self._lin(o, p + ".to_out.0")

    def _transformer(self, x, ctx, p, depth):
        B, C, H, W = x.shape
        h = self._gn(x, p + ".norm", 1e-6).permute(0, 2, 3, 1).reshape(B, H * W, C)
        h = self._lin(h, p + ".proj_in")
        for k in range(depth):
            b = f"{p}.transformer_blocks.{k}"
            n = self._ln(h, b + ".norm1")
            h = h + self._attention(n, n, b + ".attn1")
            h = h + self._attention(self._ln(h, b + ".norm2"), ctx, b + ".attn2")
            val, gate = self._lin(self._ln(h, b + ".norm3"), b + ".ff.net.0.proj").chunk(2, -1)
            h = h + self._lin(val * F.gelu(gate.float()).to(val.dtype), b + ".ff.net.2")
        h = self._lin(h, p + ".proj_out")
        return x + h.reshape(B, H, W, C).permute(0, 3, 1, 2)

    def forward_grad(self, x, timestep, context, pooled, time_ids):
        """x [B, 4, h, w] (already input-scaled), timestep [B], context [B, 77, 2048], pooled [B, 1280], time_ids [B, 6]
        (original h, w, crop top, left, target h, w) -> predicted noise [B, 4, h, w]."""
        cfg = self.cfg
        dev, dt = self.device, self.dtype
        x, context = x.to(dev, dt), context.to(dev, dt)
        if cfg.encoder_hid_dim:
            context = self._lin(context, "encoder_hid_proj")
        B = x.shape[0]
        t_emb = timestep_embedding(timestep.to(dev).float(), cfg.block_out_channels[0], time_factor=1.0).to(dt)
        emb = self._lin(F.silu(self._lin(t_emb, "time_embedding.linear_1").float()).to(dt), "time_embedding.linear_2")
        ids = timestep_embedding(time_ids.to(dev).float().reshape(-1), cfg.addition_time_embed_dim, time_factor=1.0)
        add = torch.cat([pooled.to(dev, dt), ids.reshape(B, -1).to(dt)], -1)
        emb = emb + self._lin(F.silu(self._lin(add, "add_embedding.linear_1").float()).to(dt), "add_embedding.linear_2")
        emb_act = F.silu(emb.float()).to(dt)
        down, up = self.plan
        h = self._conv(x, "conv_in")
        skips = [h]
        for lvl, res, depth, sampler in down:
            for j in range(len(res)):
                h = self._resnet(h, f"down_blocks.{lvl}.resnets.{j}", emb_act)
                if depth:
                    h = self._transformer(h, context, f"down_blocks.{lvl}.attentions.{j}", depth)
                skips.append(h)
            if sampler:
                h = self._conv(h, f"down_blocks.{lvl}.downsamplers.0.conv", stride=2)
                skips.append(h)
        h = self._resnet(h, "mid_block.resnets.0", emb_act)
        h = self._transformer(h, context, "mid_block.attentions.0", cfg.transformer_layers_per_block[-1])
        h = self._resnet(h, "mid_block.resnets.1", emb_act)
        for i, (lvl, res, depth, sampler) in enumerate(up):
            for j in range(len(res)):
                h = self._resnet(torch.cat([h, skips.pop()], 1), f"up_blocks.{i}.resnets.{j}", emb_act)
                if depth:
                    h = self._transformer(h, context, f"up_blocks.{i}.attentions.{j}", depth)
            if sampler:
                h = self._conv(F.interpolate(h, scale_factor=2, mode="nearest"), f"up_blocks.{i}.upsamplers.0.conv")
        return self._conv(self._gn(h, "conv_norm_out", 1e-5, silu=True), "conv_out")

    @torch.no_grad()
    def forward(self, x, timestep, context, pooled, time_ids):
        return self.forward_grad(x, timestep, context, pooled, time_ids)
