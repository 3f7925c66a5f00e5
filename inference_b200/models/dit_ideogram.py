"""Ideogram 4 single-stream DiT (parity: candle-gen-ideogram/src/transformer/{model,block,mrope}.rs, config.rs).

One token sequence carries the prompt and the image: prompt rows hold language-model features (13 hidden layers of
Qwen3-VL interleaved on the feature axis, 53248 wide; RMS-normed and projected), image rows hold 128-channel packed
latents (projected), and a learned per-role embedding is added (role 2 = output image, 3 = language token). Blocks are
sandwich-normed like Z-Image: x += tanh(gate) * rms2(f(rms1(x) * (1 + scale))) for attention (fused qkv, per-head q/k
RMS norm, half-rotation rotary with three interleaved position axes, 18 heads of 256) and SwiGLU; the four modulation
vectors of a block come from a per-block linear of a shared 512-wide timestep code. A segment mask keeps tokens of
different segments apart. The final layer is LayerNorm * (1 + scale) -> linear; only image rows are read out.

One implementation for both backends (nn_dual): fp32 on CPU; bf16 on a CUDA device with projections on the tcgen05
GEMM (256-wide heads run the framework's attention call: the flash kernel here is built for heads up to 128)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import nn_dual as nd

OUTPUT_IMAGE, LLM_TOKEN = 2, 3
IMAGE_POSITION_OFFSET = 65536


@dataclass
class IdeogramConfig:
    emb_dim: int = 4608
    num_layers: int = 34
    num_heads: int = 18
    mlp_dim: int = 12288
    adaln_dim: int = 512
    in_channels: int = 128
    llm_features_dim: int = 53248
    mrope_section: tuple[int, int, int] = (24, 20, 20)
    rope_theta: float = 5_000_000.0
    norm_eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.emb_dim // self.num_heads

    @staticmethod
    def from_json(j: dict) -> "IdeogramConfig":
        d = {k: j[k] for k in IdeogramConfig.__dataclass_fields__ if k in j}
        if "mrope_section" in d:
            d["mrope_section"] = tuple(d["mrope_section"])
        return IdeogramConfig(**d)


def random_ideogram_weights(cfg: IdeogramConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    E, hd = cfg.emb_dim, cfg.head_dim
    lin(w, "input_proj", E, cfg.in_channels, std)
    w["llm_cond_norm.weight"] = 1.0 + rn(cfg.llm_features_dim) * 0.1
    lin(w, "llm_cond_proj", E, cfg.llm_features_dim, std)
    lin(w, "t_embedding.mlp_in", E, E, std)
    lin(w, "t_embedding.mlp_out", E, E, std)
    lin(w, "adaln_proj", cfg.adaln_dim, E, std)
    w["embed_image_indicator.weight"] = rn(2, E) * 0.1
    for i in range(cfg.num_layers):
        p = f"layers.{i}"
        lin(w, p + ".attention.qkv", 3 * E, E, std, bias=False)
        lin(w, p + ".attention.o", E, E, std, bias=False)
        w[p + ".attention.norm_q.weight"], w[p + ".attention.norm_k.weight"] = 1.0 + rn(hd) * 0.1, 1.0 + rn(hd) * 0.1
        for n in ("w1", "w3"):
            lin(w, f"{p}.feed_forward.{n}", cfg.mlp_dim, E, std, bias=False)
        lin(w, p + ".feed_forward.w2", E, cfg.mlp_dim, std, bias=False)
        lin(w, p + ".adaln_modulation", 4 * E, cfg.adaln_dim, std)
        for n in ("attention_norm1", "attention_norm2", "ffn_norm1", "ffn_norm2"):
            w[f"{p}.{n}.weight"] = 1.0 + rn(E) * 0.1
    lin(w, "final_layer.adaln_modulation", E, cfg.adaln_dim, std)
    lin(w, "final_layer.linear", cfg.in_channels, E, std)
    return w


def packing(num_text: int, grid_h: int, grid_w: int):
    """(position_ids [S, 3], indicator [S]) of the packed sequence [prompt rows, image rows]: prompt row i sits at
    (i, i, i), image cell (h, w) at (65536, 65536 + h, 65536 + w)."""
    t = torch.arange(num_text)
    txt = torch.stack((t, t, t), dim=1)
    h = torch.arange(grid_h)[:, None].expand(grid_h, grid_w).reshape(-1) + IMAGE_POSITION_OFFSET
    w_ = torch.arange(grid_w)[None, :].expand(grid_h, grid_w).reshape(-1) + IMAGE_POSITION_OFFSET
    img = torch.stack((torch.full_like(h, IMAGE_POSITION_OFFSET), h, w_), dim=1)
    ind = torch.cat([torch.full((num_text,), LLM_TOKEN), torch.full((grid_h * grid_w,), OUTPUT_IMAGE)])
    return torch.cat([txt, img]).float(), ind


def mrope_tables(position_ids: torch.Tensor, head_dim: int, theta: float, section: tuple[int, int, int]):
    """position_ids [S, 3] -> cos, sin [S, head_dim / 2]. Frequency d belongs to the row axis when d % 3 == 1 (below
    3 * section[1]), to the column axis when d % 3 == 2 (below 3 * section[2]), else to the first axis."""
    half = head_dim // 2
    d = torch.arange(half)
    inv = theta ** (-(2.0 * d.double()) / head_dim)
    axis = torch.zeros(half, dtype=torch.long)
    axis[(d % 3 == 1) & (d < section[1] * 3)] = 1
    axis[(d % 3 == 2) & (d < section[2] * 3)] = 2
    ang = position_ids.double()[:, axis] * inv[None, :]
    return ang.cos().float(), ang.sin().float()


class IdeogramDiT:
    def __init__(self, cfg: IdeogramConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.bag = nd.WeightBag(weights, dtype, device)
        self.dtype, self.device = self.bag.dtype, self.bag.device
        self._cache = None

    def weight_bytes(self) -> int:
        return self.bag.nbytes()

    def _t_embedding(self, t: torch.Tensor) -> torch.Tensor:
        half = self.cfg.emb_dim // 2
        f = torch.exp(-(math.log(1e4) / (half - 1)) * torch.arange(half, dtype=torch.float32, device=self.device))
        ang = (t.to(self.device).float() * 1e4)[:, None] * f[None]
        e = torch.cat([ang.sin(), ang.cos()], -1).to(self.dtype)
        return self.bag.lin(self.bag.lin(e, "t_embedding.mlp_in", act="silu"), "t_embedding.mlp_out")

    def _prepared(self, position_ids, segment_ids, indicator):
        key = (position_ids.shape, float(position_ids.sum()), int(indicator.sum()),
               None if segment_ids is None else int(segment_ids.sum()))
        if self._cache is None or self._cache[0] != key:
            cfg = self.cfg
            cos, sin = mrope_tables(position_ids, cfg.head_dim, cfg.rope_theta, cfg.mrope_section)
            ind = indicator.to(self.device)
            mask = None
            if segment_ids is not None and bool((segment_ids != segment_ids[0]).any()):
                s = segment_ids.to(self.device)
                mask = torch.zeros(len(s), len(s), device=self.device, dtype=self.dtype)
                mask.masked_fill_(s[:, None] != s[None, :], float("-inf"))
                mask = mask[None, None]
            self._cache = (key, (ind == LLM_TOKEN).to(self.dtype)[None, :, None], (ind == OUTPUT_IMAGE).to(self.dtype)[None, :, None],
                           (ind == OUTPUT_IMAGE).long()[None], cos.to(self.device), sin.to(self.device), mask)
        return self._cache[1:]

    def forward_grad(self, llm_features: torch.Tensor, x: torch.Tensor, t: torch.Tensor, position_ids: torch.Tensor,
                     indicator: torch.Tensor, segment_ids: torch.Tensor | None = None) -> torch.Tensor:
        """llm_features [B, S, llm_features_dim] (zeros on image rows), x [B, S, in_channels] (zeros on prompt rows),
        t [B] in (0, 1) (0 = noise), position_ids [S, 3], indicator [S] -> [B, S, in_channels] (fp32)."""
        cfg, dev, dt = self.cfg, self.device, self.dtype
        llm_mask, img_mask, img_idx, cos, sin, mask = self._prepared(position_ids, segment_ids, indicator)
        B, S, _ = x.shape
        E, nh, hd = cfg.emb_dim, cfg.num_heads, cfg.head_dim
        h = self.bag.lin(x.to(dev, dt) * img_mask, "input_proj") * img_mask
        ada = F.silu(self.bag.lin(self._t_embedding(t)[:, None, :], "adaln_proj").float()).to(dt)           # [B, 1, adaln]
        llm = nd.rms_norm(llm_features.to(dev, dt) * llm_mask, self.bag["llm_cond_norm.weight"], 1e-6)
        h = h + self.bag.lin(llm, "llm_cond_proj") * llm_mask
        h = h + self.bag["embed_image_indicator.weight"][img_idx.expand(B, S)]
        for i in range(cfg.num_layers):
            p = f"layers.{i}"
            m = self.bag.lin(ada, p + ".adaln_modulation").chunk(4, dim=-1)
            sc_a, g_a, sc_m, g_m = 1 + m[0], torch.tanh(m[1].float()).to(dt), 1 + m[2], torch.tanh(m[3].float()).to(dt)
            n = nd.rms_norm(h, self.bag[p + ".attention_norm1.weight"], cfg.norm_eps) * sc_a
            qkv = self.bag.lin(n, p + ".attention.qkv").reshape(B, S, 3, nh, hd)
            q = nd.rope_half(nd.rms_norm(qkv[:, :, 0], self.bag[p + ".attention.norm_q.weight"], 1e-5), cos, sin)
            k = nd.rope_half(nd.rms_norm(qkv[:, :, 1], self.bag[p + ".attention.norm_k.weight"], 1e-5), cos, sin)
            o = self.bag.lin(nd.attention(q, k, qkv[:, :, 2], mask=mask), p + ".attention.o")
            h = h + nd.rms_norm(o, self.bag[p + ".attention_norm2.weight"], cfg.norm_eps) * g_a
            n = nd.rms_norm(h, self.bag[p + ".ffn_norm1.weight"], cfg.norm_eps) * sc_m
            f = p + ".feed_forward."
            ff = self.bag.lin((F.silu(self.bag.lin(n, f + "w1").float()) * self.bag.lin(n, f + "w3").float()).to(dt), f + "w2")
            h = h + nd.rms_norm(ff, self.bag[p + ".ffn_norm2.weight"], cfg.norm_eps) * g_m
        scale = 1 + self.bag.lin(F.silu(ada.float()).to(dt), "final_layer.adaln_modulation")
        return self.bag.lin(nd.layer_norm(h, eps=1e-6) * scale, "final_layer.linear").float()

    @torch.no_grad()
    def forward(self, llm_features, x, t, position_ids, indicator, segment_ids=None):
        return self.forward_grad(llm_features, x, t, position_ids, indicator, segment_ids)


# ---- sampling schedule ------------------------------------------------------------------------------------------------
def _ndtri(p: float) -> float:
    """Inverse of the standard normal CDF (rational approximation, relative error below 1.2e-9)."""
    if p <= 0.0:
        return float("-inf")
    if p >= 1.0:
        return float("inf")
    a = (-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02, 1.38357751867269e+02,
         -3.066479806614716e+01, 2.506628277459239e+00)
    b = (-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02, 6.680131188771972e+01,
         -1.328068155288572e+01)
    c = (-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00, -2.549732539343734e+00,
         4.374664141464968e+00, 2.938163982698783e+00)
    d = (7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00, 3.754408661907416e+00)
    lo = 0.02425
    if p < lo or p > 1.0 - lo:
        q = math.sqrt(-2.0 * math.log(p if p < lo else 1.0 - p))
        v = (((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) / \
            ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1.0)
        return v if p < lo else -v
    q = p - 0.5
    r = q * q
    return (((((a[0] * r + a[1]) * r + a[2]) * r + a[3]) * r + a[4]) * r + a[5]) * q / \
        (((((b[0] * r + b[1]) * r + b[2]) * r + b[3]) * r + b[4]) * r + 1.0)


def logit_normal_time(u: float, height: int, width: int, known_mean: float, std: float) -> float:
    """Model time (0 = noise, 1 = image) at fraction u of the schedule: a logit-normal quantile whose mean grows with
    half the log of the pixel count relative to 512 x 512, clamped to the trained range."""
    mean = known_mean + 0.5 * math.log(height * width / (512.0 * 512.0))
    y = mean + std * _ndtri(u)
    mapped = 1.0 - 1.0 / (1.0 + math.exp(-y))
    t_min, t_max = 1.0 / (1.0 + math.exp(0.5 * 18.0)), 1.0 / (1.0 + math.exp(0.5 * -15.0))
    return min(max(mapped, t_min), t_max)


def preset_mu_std(num_steps: int) -> tuple[float, float]:
    return (0.5, 1.75) if num_steps <= 15 else ((0.0, 1.75) if num_steps <= 33 else (0.0, 1.5))
