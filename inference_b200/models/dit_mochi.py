"""Mochi 1 video model: the asymmetric dual-stream DiT and the asymmetric causal-conv video decoder
(parity: candle-gen-mochi/src/transformer.rs, rope.rs, vae.rs, conv3d.rs, nn.rs).

DiT: a 3072-wide visual stream (24 heads of 128) and a 1536-wide text stream attend jointly; each block modulates both
streams from the timestep code with weight-free RMS norms: x += tanh(gate) * rms(f(rms(x) * (1 + scale))). The last
block only reads the text stream. The timestep code is a sinusoid MLP plus an attention-pooled summary of the T5
states. Rotary angles are LEARNED: positions (frame index, centred row / column coordinates scaled to a 192 x 192
reference area) times a [3, heads, 64] frequency tensor, applied to adjacent pairs.

Padding never reaches this module: the caller passes the valid T5 rows only, which is what masking padded keys in the
joint attention and in the pooler computes for every row that is read afterwards.

Decoder: 1x1x1 conv in, residual blocks of causal 3x3x3 convolutions (front-padded in time with the first frame,
edge-padded in space, GroupNorm per frame), three up blocks that widen by a linear and rearrange depth to time / space
(1x2x2, 2x2x2, 3x2x2), SiLU, linear to RGB; the first (6 - 1) output frames are dropped. fp32 throughout.

One implementation for both backends (nn_dual)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from . import nn_dual as nd

QK_NORM_EPS = 1e-5
BASE_AREA = 192.0 * 192.0


@dataclass
class MochiConfig:
    patch_size: int = 2
    num_heads: int = 24
    head_dim: int = 128
    num_layers: int = 48
    pooled_dim: int = 1536
    in_channels: int = 12
    text_embed_dim: int = 4096
    time_embed_dim: int = 256
    pool_heads: int = 8
    eps: float = 1e-6

    @property
    def inner(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def ff_inner(self) -> int:
        return (self.inner * 4 * 2) // 3

    @property
    def ff_ctx_inner(self) -> int:
        return (self.pooled_dim * 4 * 2) // 3

    @staticmethod
    def from_json(j: dict) -> "MochiConfig":
        return MochiConfig(**{k: j[k] for k in MochiConfig.__dataclass_fields__ if k in j})


def random_mochi_weights(cfg: MochiConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    D, Pd, p = cfg.inner, cfg.pooled_dim, cfg.patch_size
    w["patch_embed.proj.weight"] = rn(D, cfg.in_channels, p, p) * std
    w["patch_embed.proj.bias"] = rn(D) * std
    w["pos_frequencies"] = rn(3, cfg.num_heads, cfg.head_dim // 2) * 0.3
    lin(w, "time_embed.timestep_embedder.linear_1", D, cfg.time_embed_dim, std)
    lin(w, "time_embed.timestep_embedder.linear_2", D, D, std)
    E = cfg.text_embed_dim
    lin(w, "time_embed.pooler.to_kv", 2 * E, E, std)
    lin(w, "time_embed.pooler.to_q", E, E, std)
    lin(w, "time_embed.pooler.to_out", D, E, std)
    lin(w, "time_embed.caption_proj", Pd, E, std)
    for i in range(cfg.num_layers):
        b, last = f"transformer_blocks.{i}", i == cfg.num_layers - 1
        lin(w, b + ".norm1.linear", 4 * D, D, std)
        lin(w, b + (".norm1_context.linear_1" if last else ".norm1_context.linear"), Pd if last else 4 * Pd, D, std)
        a = b + ".attn1."
        for n in ("to_q", "to_k", "to_v"):
            lin(w, a + n, D, D, std, bias=False)
        for n in ("add_q_proj", "add_k_proj", "add_v_proj"):
            lin(w, a + n, D, Pd, std, bias=False)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            w[a + n + ".weight"] = 1.0 + rn(cfg.head_dim) * 0.1
        lin(w, a + "to_out.0", D, D, std)
        lin(w, b + ".ff.net.0.proj", 2 * cfg.ff_inner, D, std, bias=False)
        lin(w, b + ".ff.net.2", D, cfg.ff_inner, std, bias=False)
        if not last:
            lin(w, a + "to_add_out", Pd, D, std)
            lin(w, b + ".ff_context.net.0.proj", 2 * cfg.ff_ctx_inner, Pd, std, bias=False)
            lin(w, b + ".ff_context.net.2", Pd, cfg.ff_ctx_inner, std, bias=False)
    lin(w, "norm_out.linear", 2 * D, D, std)
    lin(w, "proj_out", p * p * cfg.in_channels, D, std)
    return w


def mochi_positions(frames: int, height: int, width: int) -> torch.Tensor:
    """[frames * height * width, 3]: (frame, row centre, column centre); the spatial grid is rescaled so that its
    area equals 192 x 192 and centred on zero."""
    scale = math.sqrt(BASE_AREA / (height * width))

    def centres(n):
        lo, hi = -n * scale / 2.0, n * scale / 2.0
        step = (hi - lo) / n
        return torch.tensor([(lo + step * k + lo + step * (k + 1)) / 2.0 for k in range(n)], dtype=torch.float32)

    t = torch.arange(frames, dtype=torch.float32)
    g = torch.stack(torch.meshgrid(t, centres(height), centres(width), indexing="ij"), dim=-1)
    return g.reshape(-1, 3)


def rope_per_head(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Adjacent-pair rotation with per-head angles: x [B, S, H, D], cos / sin [S, H, D / 2]."""
    B, S, H, D = x.shape
    xr = x.float().reshape(B, S, H, D // 2, 2)
    e, o = xr[..., 0], xr[..., 1]
    return torch.stack((e * cos - o * sin, e * sin + o * cos), dim=-1).reshape(B, S, H, D).to(x.dtype)


class MochiDiT:
    def __init__(self, cfg: MochiConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        w = dict(weights)
        pw = w.pop("patch_embed.proj.weight")
        w["patch_embed.proj.weight"] = pw.reshape(pw.shape[0], -1)             # conv with stride = kernel = a linear
        self.bag = nd.WeightBag(w, dtype, device, keep_fp32=("pos_frequencies",))
        self.dtype, self.device = self.bag.dtype, self.bag.device
        self._rope = None

    def weight_bytes(self) -> int:
        return self.bag.nbytes()

    def _rope_tables(self, f, ph, pw):
        if self._rope is None or self._rope[0] != (f, ph, pw):
            pf = self.bag["pos_frequencies"].float()
            ang = (mochi_positions(f, ph, pw).to(self.device) @ pf.reshape(3, -1)).reshape(-1, pf.shape[1], pf.shape[2])
            self._rope = ((f, ph, pw), ang.cos(), ang.sin())
        return self._rope[1], self._rope[2]

    def _rmsn(self, x):
        return nd.rms_norm(x, None, self.cfg.eps)

    def _swiglu(self, x, name):
        a, b = self.bag.lin(x, name + ".net.0.proj").float().chunk(2, dim=-1)
        return self.bag.lin((a * F.silu(b)).to(self.dtype), name + ".net.2")

    def conditioning(self, enc: torch.Tensor, timestep: torch.Tensor):
        """enc [B, L, text_embed_dim] (valid rows only), timestep [B] -> (timestep code [B, inner], text stream
        [B, L, pooled_dim])."""
        cfg, dt = self.cfg, self.dtype
        enc = enc.to(self.device, dt)
        B, L, E = enc.shape
        tp = nd.sinusoidal_embedding(timestep.to(self.device), cfg.time_embed_dim).to(dt)
        te = self.bag.lin(self.bag.lin(tp, "time_embed.timestep_embedder.linear_1", act="silu"),
                          "time_embed.timestep_embedder.linear_2")
        pool = enc.float().mean(1, keepdim=True).to(dt)
        kv = self.bag.lin(torch.cat([pool, enc], 1), "time_embed.pooler.to_kv").reshape(B, L + 1, 2, cfg.pool_heads, -1)
        q = self.bag.lin(pool, "time_embed.pooler.to_q").reshape(B, 1, cfg.pool_heads, -1)
        pooled = self.bag.lin(nd.attention(q, kv[:, :, 0], kv[:, :, 1]), "time_embed.pooler.to_out")[:, 0]
        return te + pooled, self.bag.lin(enc, "time_embed.caption_proj")

    def forward_grad(self, hidden: torch.Tensor, enc: torch.Tensor, timestep: torch.Tensor) -> torch.Tensor:
        """hidden [B, C, F, H, W], enc [B, L, 4096] (valid rows), timestep [B] -> velocity [B, C, F, H, W] (fp32)."""
        cfg, dt = self.cfg, self.dtype
        B, C, Fr, H, W = hidden.shape
        p, nh, hd, D = cfg.patch_size, cfg.num_heads, cfg.head_dim, cfg.inner
        ph, pw = H // p, W // p
        temb, txt = self.conditioning(enc, timestep)
        st = F.silu(temb.float()).to(dt)[:, None, :]
        x = hidden.to(self.device, dt).permute(0, 2, 1, 3, 4).reshape(B * Fr, C, H, W)
        hs = self.bag.lin(nd.patchify(x, p), "patch_embed.proj").reshape(B, Fr * ph * pw, D)
        cos, sin = self._rope_tables(Fr, ph, pw)
        Sv, St = hs.shape[1], txt.shape[1]
        heads = lambda t: t.reshape(B, -1, nh, hd)       # noqa: E731
        for i in range(cfg.num_layers):
            b, last = f"transformer_blocks.{i}", i == cfg.num_layers - 1
            a = b + ".attn1."
            sa, ga, sm, gm = self.bag.lin(st, b + ".norm1.linear").chunk(4, dim=-1)
            nh_ = self._rmsn(hs) * (1 + sa)
            if last:
                ne = self._rmsn(txt) * (1 + self.bag.lin(st, b + ".norm1_context.linear_1"))
            else:
                esa, ega, esm, egm = self.bag.lin(st, b + ".norm1_context.linear").chunk(4, dim=-1)
                ne = self._rmsn(txt) * (1 + esa)
            q = rope_per_head(nd.rms_norm(heads(self.bag.lin(nh_, a + "to_q")), self.bag[a + "norm_q.weight"], QK_NORM_EPS), cos, sin)
            k = rope_per_head(nd.rms_norm(heads(self.bag.lin(nh_, a + "to_k")), self.bag[a + "norm_k.weight"], QK_NORM_EPS), cos, sin)
            v = heads(self.bag.lin(nh_, a + "to_v"))
            eq = nd.rms_norm(heads(self.bag.lin(ne, a + "add_q_proj")), self.bag[a + "norm_added_q.weight"], QK_NORM_EPS)
            ek = nd.rms_norm(heads(self.bag.lin(ne, a + "add_k_proj")), self.bag[a + "norm_added_k.weight"], QK_NORM_EPS)
            ev = heads(self.bag.lin(ne, a + "add_v_proj"))
            o = nd.attention(torch.cat([q, eq], 1), torch.cat([k, ek], 1), torch.cat([v, ev], 1))
            hs = hs + self._rmsn(self.bag.lin(o[:, :Sv], a + "to_out.0")) * torch.tanh(ga.float()).to(dt)
            hs = hs + self._rmsn(self._swiglu(self._rmsn(hs) * (1 + sm), b + ".ff")) * torch.tanh(gm.float()).to(dt)
            if not last:
                txt = txt + self._rmsn(self.bag.lin(o[:, Sv:], a + "to_add_out")) * torch.tanh(ega.float()).to(dt)
                txt = txt + self._rmsn(self._swiglu(self._rmsn(txt) * (1 + esm), b + ".ff_context")) * torch.tanh(egm.float()).to(dt)
        scale, shift = self.bag.lin(st, "norm_out.linear").chunk(2, dim=-1)
        out = self.bag.lin(nd.layer_norm(hs, eps=1e-6) * (1 + scale) + shift, "proj_out").float()
        return out.reshape(B, Fr, ph, pw, p, p, C).permute(0, 6, 1, 2, 4, 3, 5).reshape(B, C, Fr, H, W)

    @torch.no_grad()
    def forward(self, hidden, enc, timestep):
        return self.forward_grad(hidden, enc, timestep)


# ---- decoder ------------------------------------------------------------------------------------------------------------
MOCHI_LATENTS_MEAN = (-0.06730895953510081, -0.038011381506090416, -0.07477820912866141, -0.05565264470995561,
                      0.012767231469026969, -0.04703542746246419, 0.043896967884726704, -0.09346305707025976,
                      -0.09918314763016893, -0.008729793427399178, -0.011931556316503654, -0.0321993391887285)
MOCHI_LATENTS_STD = (0.9263795028493863, 0.9248894543193766, 0.9393059390890617, 0.959253732819592, 0.8244560132752793,
                     0.917259975397747, 0.9294154431013696, 1.3720942357788521, 0.881393668867029, 0.9168315692124348,
                     0.9185249279345552, 0.9274757570805041)


@dataclass
class MochiVaeConfig:
    latent_channels: int = 12
    out_channels: int = 3
    decoder_block_out_channels: tuple[int, ...] = (128, 256, 512, 768)
    layers_per_block: tuple[int, ...] = (3, 3, 4, 6, 3)
    temporal_expansions: tuple[int, ...] = (1, 2, 3)
    spatial_expansions: tuple[int, ...] = (2, 2, 2)
    latents_mean: tuple[float, ...] = MOCHI_LATENTS_MEAN
    latents_std: tuple[float, ...] = MOCHI_LATENTS_STD
    scaling_factor: float = 1.0
    groups: int = 32

    @property
    def temporal_ratio(self) -> int:
        return math.prod(self.temporal_expansions)

    @property
    def spatial_ratio(self) -> int:
        return math.prod(self.spatial_expansions)

    @staticmethod
    def from_json(j: dict) -> "MochiVaeConfig":
        d = {k: (tuple(j[k]) if isinstance(j[k], list) else j[k]) for k in MochiVaeConfig.__dataclass_fields__ if k in j}
        return MochiVaeConfig(**d)


def _vae_layout(cfg: MochiVaeConfig):
    """[(prefix, channels, resnets, up-projection (out_ch, t, s) or None)] in execution order."""
    ch, lp = cfg.decoder_block_out_channels, cfg.layers_per_block
    n, k = len(ch), len(cfg.temporal_expansions)
    out = [("block_in", ch[-1], lp[-1], None)]
    for i in range(n - 1):
        out.append((f"up_blocks.{i}", ch[n - 1 - i], lp[len(lp) - 2 - i],
                    (ch[n - 2 - i], cfg.temporal_expansions[k - 1 - i], cfg.spatial_expansions[k - 1 - i])))
    out.append(("block_out", ch[0], lp[0], None))
    return out


def random_mochi_vae_weights(cfg: MochiVaeConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    rn, _ = nd.randn_weights(seed)
    w = {"conv_in.weight": rn(cfg.decoder_block_out_channels[-1], cfg.latent_channels, 1, 1, 1) * 0.3,
         "conv_in.bias": rn(cfg.decoder_block_out_channels[-1]) * 0.02}
    for pre, c, nres, up in _vae_layout(cfg):
        for r in range(nres):
            for j in (1, 2):
                w[f"{pre}.resnets.{r}.norm{j}.norm_layer.weight"] = 1.0 + rn(c) * 0.05
                w[f"{pre}.resnets.{r}.norm{j}.norm_layer.bias"] = rn(c) * 0.02
                w[f"{pre}.resnets.{r}.conv{j}.conv.weight"] = rn(c, c, 3, 3, 3) / math.sqrt(27 * c) * 0.7
                w[f"{pre}.resnets.{r}.conv{j}.conv.bias"] = rn(c) * 0.02
        if up is not None:
            oc, t, s = up
            w[f"{pre}.proj.weight"] = rn(oc * t * s * s, c) / math.sqrt(c)
            w[f"{pre}.proj.bias"] = rn(oc * t * s * s) * 0.02
    w["proj_out.weight"] = rn(cfg.out_channels, cfg.decoder_block_out_channels[0]) / math.sqrt(cfg.decoder_block_out_channels[0])
    w["proj_out.bias"] = rn(cfg.out_channels) * 0.02
    return {"decoder." + k: v for k, v in w.items()}


class MochiVaeDecoder:
    """latents [B, 12, T, H/8, W/8] (the DiT's normalised space) -> video [B, 3, (T - 1) * 6 + 1, H, W] in ~[-1, 1]."""

    def __init__(self, cfg: MochiVaeConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = {k[len("decoder."):]: v.to(self.device, dtype).contiguous() for k, v in weights.items()
                  if k.startswith("decoder.")}
        c = cfg.latent_channels
        self.mean = torch.tensor(cfg.latents_mean, dtype=dtype, device=self.device).view(1, c, 1, 1, 1)
        self.std = torch.tensor(cfg.latents_std, dtype=dtype, device=self.device).view(1, c, 1, 1, 1)

    def _conv(self, x, name, cache):
        w, b = self.w[name + ".weight"], self.w[name + ".bias"]
        kt, kh, kw = w.shape[2:]
        if kt > 1:
            prev = cache.get(name) if cache is not None else None
            front = prev if prev is not None else x[:, :, :1].expand(-1, -1, kt - 1, -1, -1)
            x = torch.cat([front, x], dim=2)
            if cache is not None:
                cache[name] = x[:, :, -(kt - 1):].clone()
        if kh > 1 or kw > 1:
            B, C, T, H, W = x.shape
            x = F.pad(x.reshape(B, C * T, H, W), ((kw - 1) // 2,) * 2 + ((kh - 1) // 2,) * 2, mode="replicate")
            x = x.reshape(B, C, T, H + kh - 1, W + kw - 1)
        return F.conv3d(x, w, b)

    def _gn(self, x, name):
        B, C, T, H, W = x.shape
        y = F.group_norm(x.transpose(1, 2).reshape(B * T, C, H, W), self.cfg.groups, self.w[name + ".norm_layer.weight"],
                         self.w[name + ".norm_layer.bias"], 1e-5)
        return y.reshape(B, T, C, H, W).transpose(1, 2)

    def _body(self, x, cache):
        x = self._conv(x.to(self.device, self.dtype), "conv_in", cache)
        for pre, c, nres, up in _vae_layout(self.cfg):
            for r in range(nres):
                p = f"{pre}.resnets.{r}"
                h = self._conv(F.silu(self._gn(x, p + ".norm1")), p + ".conv1.conv", cache)
                x = x + self._conv(F.silu(self._gn(h, p + ".norm2")), p + ".conv2.conv", cache)
            if up is not None:
                oc, st, ss = up
                y = F.linear(x.permute(0, 2, 3, 4, 1), self.w[pre + ".proj.weight"], self.w[pre + ".proj.bias"])
                B, T, H, W, _ = y.shape
                x = y.reshape(B, T, H, W, oc, st, ss, ss).permute(0, 4, 1, 5, 2, 6, 3, 7).reshape(B, oc, T * st, H * ss, W * ss)
        y = F.linear(F.silu(x).permute(0, 2, 3, 4, 1), self.w["proj_out.weight"], self.w["proj_out.bias"])
        return y.permute(0, 4, 1, 2, 3)

    @torch.no_grad()
    def decode(self, latents: torch.Tensor, chunk_frames: int | None = None) -> torch.Tensor:
        """`chunk_frames`: decode that many latent frames at a time, carrying each causal convolution's last two
        input frames between chunks (same result, bounded activation memory)."""
        z = latents.to(self.device, self.dtype) * self.std / self.cfg.scaling_factor + self.mean
        drop = self.cfg.temporal_ratio - 1
        T = z.shape[2]
        if chunk_frames is None or chunk_frames >= T:
            v = self._body(z, None)
            return v[:, :, drop:] if v.shape[2] >= self.cfg.temporal_ratio else v
        cache: dict = {}
        parts = []
        for s in range(0, T, max(1, chunk_frames)):
            v = self._body(z[:, :, s:s + max(1, chunk_frames)], cache)
            parts.append(v[:, :, drop:] if (s == 0 and v.shape[2] >= self.cfg.temporal_ratio) else v)
        return torch.cat(parts, dim=2)


def linear_quadratic_sigmas(num_steps: int, threshold_noise: float = 0.025) -> list[float]:
    """Noise levels 1 -> ~0 (no terminal zero): the first half of the steps removes `threshold_noise` linearly, the
    second half follows the quadratic that continues it to zero noise one step past the end."""
    n, ls = float(num_steps), num_steps // 2
    sched = [i * threshold_noise / ls for i in range(ls)]
    diff = ls - threshold_noise * n
    qs = float(num_steps - ls)
    qc = diff / (ls * qs * qs)
    lc = threshold_noise / ls - 2.0 * diff / (qs * qs)
    const = qc * ls * ls
    sched += [qc * i * i + lc * i + const for i in range(ls, num_steps)]
    return [1.0 - x for x in sched]
