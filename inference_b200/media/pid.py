"""PiD (Pixel Diffusion Decoder): an optional, super-resolving replacement for a generator's VAE decode.

PiD denoises directly in pixel space at `sr_scale` times the latent's natural resolution, conditioned on the generation's
caption and on the (possibly still noisy) latent: a 4-step distilled student decodes and upsamples in one pass. It is tied to
a latent space, not to a model: one topology serves every generator, parameterised per latent space by a checkpoint, a
channel count and a latent normalisation.

Behaviour follows the reference's candle-gen-pid crate:
  - registry.rs:1-140        latent spaces (qwenimage, flux / zimage, sd3, sdxl, flux2), their channels, norms and scale
  - config.rs:1-140          the sr4x and sr4x-v1.5 configurations; the 4-step student schedule
  - backbone/mod.rs:1-208    PixDiT: patch-level MMDiT blocks over (image patches, caption), then pixel-level blocks
                             conditioned per patch; layers.rs, blocks.rs, rope.rs: the layers, NTK-scaled 2-D rotary phases
  - lq.rs:1-398              the low-quality-latent adapter: convolution trunk, per-block heads, sigma-aware gates, the
                             v1.5 pixel-stage injection
  - sampler.rs:1-209         the student's SDE / ODE sampler over velocity predictions
  - tiling.rs:1-236          overlapping tiles with feathered blending for large outputs; budget.rs: tile planning
  - caption.rs:1-169         Gemma-2 caption states: instruction prefix + caption, position 0 and the last 299 positions
  - engine.rs:1-577          load-once / decode-many engine, v1.0 / v1.5 detection from the weights, early-stop capture

One implementation for both backends on `models.nn_dual`: fp32 on the oracle backend; on the device the projections run on
the tcgen05 GEMM and attention over 64-wide heads on the 64-wide tcgen05 attention kernel.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field, replace
from pathlib import Path

import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..models import nn_dual as nd

RMS_EPS, GN_EPS, GN_GROUPS = 1e-6, 1e-5, 4
ROPE_THETA, ROPE_SCALE = 10000.0, 16.0
PIXEL_POS_TRAIN_MAX = 3840.0
MODEL_MAX_LENGTH, PAD_ID = 300, 0
GEMMA_MERGED_FILE = "gemma-2-2b-it.safetensors"
TILE_ALIGN, MIN_TILE_EDGE, DEFAULT_TILE_OVERLAP, PREFERRED_TILE_EDGE = 512, 1024, 256, 2048
CHI_PROMPT = ('Given a user prompt, generate an "Enhanced prompt" that provides detailed visual descriptions suitable for image '
              "generation. Evaluate the level of detail in the user prompt:\n- If the prompt is simple, focus on adding specifics "
              "about colors, shapes, sizes, textures, and spatial relationships to create vivid and concrete scenes.\n- If the "
              "prompt is already detailed, refine and enhance the existing details slightly without overcomplicating.\nHere are "
              "examples of how to transform or refine prompts:\n- User Prompt: A cat sleeping -> Enhanced: A small, fluffy white "
              "cat curled up in a round shape, sleeping peacefully on a warm sunny windowsill, surrounded by pots of blooming red "
              "flowers.\n- User Prompt: A busy city street -> Enhanced: A bustling city street scene at dusk, featuring glowing "
              "street lamps, a diverse crowd of people in colorful clothing, and a double-decker bus passing by towering glass "
              "skyscrapers.\nPlease generate only the enhanced description for the prompt below and avoid including any additional "
              "commentary or evaluations:\nUser Prompt: ")


# ---- registry and configuration ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class BackboneSpec:
    latent_space: str
    latent_channels: int
    latent_norm: tuple                     # ("affine", scale, shift) | ("per_channel",) | ("batch_norm",)
    latent_spatial_down_factor: int = 8
    pid_scale: int = 4
    vp_frame: bool = False
    ckpt_2k: str | None = None
    ckpt_2kto4k: str | None = None


_CK = "checkpoints/PiD_{}_sr4x_official_{}_distill_4step/model_ema_bf16.pth"
SPECS = {
    "qwenimage": BackboneSpec("qwenimage", 16, ("per_channel",), ckpt_2kto4k=_CK.format("v1pt5_res2kto4k", "qwenimage")),
    "flux": BackboneSpec("flux", 16, ("affine", 0.3611, 0.1159), ckpt_2k=_CK.format("res2k", "flux"),
                         ckpt_2kto4k=_CK.format("v1pt5_res2kto4k", "flux")),
    "sd3": BackboneSpec("sd3", 16, ("affine", 1.5305, 0.0609), ckpt_2k=_CK.format("res2k", "sd3"), ckpt_2kto4k=_CK.format("res2kto4k", "sd3")),
    "sdxl": BackboneSpec("sdxl", 4, ("affine", 0.13025, 0.0), vp_frame=True, ckpt_2kto4k=_CK.format("res2kto4k", "sdxl")),
    "flux2": BackboneSpec("flux2", 128, ("batch_norm",), latent_spatial_down_factor=16, ckpt_2k=_CK.format("res2k", "flux2"),
                          ckpt_2kto4k=_CK.format("v1pt5_res2kto4k", "flux2")),
}
ALIASES = {"qwenimage-2512": "qwenimage", "zimage": "flux", "zimage-turbo": "flux", "flux2-klein-4b": "flux2", "flux2-klein-9b": "flux2"}


def lookup(backbone: str) -> BackboneSpec | None:
    return SPECS.get(ALIASES.get(backbone, backbone))


@dataclass
class PidConfig:
    in_channels: int = 3
    num_groups: int = 24
    hidden_size: int = 1536
    pixel_hidden_size: int = 16
    pixel_attn_hidden_size: int = 1152
    pixel_num_groups: int = 16
    patch_depth: int = 14
    pixel_depth: int = 2
    patch_size: int = 16
    txt_embed_dim: int = 2304
    txt_max_length: int = 300
    text_rope_theta: float = 10000.0
    rope_ref_h: int = 1024
    rope_ref_w: int = 1024
    lq_latent_channels: int = 16
    lq_hidden_dim: int = 512
    lq_num_res_blocks: int = 4
    lq_interval: int = 2
    lq_replicate_padding: bool = False
    pit_lq_inject: bool = False
    sr_scale: int = 4
    latent_spatial_down_factor: int = 8

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_groups

    @property
    def pixel_head_dim(self) -> int:
        return self.pixel_attn_hidden_size // self.pixel_num_groups

    @property
    def num_lq_outputs(self) -> int:
        return -(-self.patch_depth // self.lq_interval)

    @staticmethod
    def sr4x() -> "PidConfig":
        return PidConfig()

    @staticmethod
    def sr4x_v1pt5() -> "PidConfig":
        return PidConfig(rope_ref_h=2048, rope_ref_w=2048, lq_hidden_dim=1024, lq_replicate_padding=True, pit_lq_inject=True)


STUDENT_T_LIST, FM_TIMESCALE = (0.999, 0.866, 0.634, 0.342, 0.0), 1000.0


def detect_v1pt5(w) -> bool:
    """Two signals that must agree: the first gate's projection has one output row (a per-token scalar gate) and the
    checkpoint carries the pixel-stage gate."""
    k = "lq_proj.gate_modules.0.content_proj.weight"
    if k not in w:
        raise LoadError("pid: not a PiD student checkpoint (no lq_proj.gate_modules.0.content_proj.weight)")
    scalar, pit = w[k].shape[0] == 1, "pit_lq_gate.content_proj.weight" in w
    if scalar != pit:
        raise LoadError(f"pid: inconsistent v1.5 signals: scalar gate = {scalar}, pixel-stage gate present = {pit}")
    return scalar


def config_for_spec(spec: BackboneSpec, v1pt5: bool, base: PidConfig | None = None) -> PidConfig:
    cfg = base if base is not None else (PidConfig.sr4x_v1pt5() if v1pt5 else PidConfig.sr4x())
    return replace(cfg, lq_latent_channels=spec.latent_channels, latent_spatial_down_factor=spec.latent_spatial_down_factor,
                   sr_scale=spec.pid_scale)


# ---- positions --------------------------------------------------------------------------------------------------------------
def rope_2d_ntk(head_dim: int, hs: int, ws: int, ref_h: int, ref_w: int, theta: float = ROPE_THETA, scale: float = ROPE_SCALE
                ) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [hs * ws, head_dim / 2]: even lanes follow the column, odd lanes the row; positions are spread over
    [0, scale]; a grid larger than the reference grid stretches theta by (grid / ref)^(d / (d - 2)) per axis, d = head_dim / 2."""
    d_axis = head_dim / 2.0
    ntk = d_axis / (d_axis - 2.0) if d_axis > 2.0 else 1.0
    th_h, th_w = theta * (hs / ref_h) ** ntk, theta * (ws / ref_w) ** ntk
    j = torch.arange(head_dim // 4, dtype=torch.float64)
    fw, fh = 1.0 / th_w ** (4 * j / head_dim), 1.0 / th_h ** (4 * j / head_dim)
    lin = lambda n: (torch.arange(n, dtype=torch.float64) * scale / (n - 1)) if n > 1 else torch.zeros(n, dtype=torch.float64)   # noqa: E731
    yp, xp = lin(hs), lin(ws)
    ang = torch.empty(hs, ws, head_dim // 2, dtype=torch.float64)
    ang[..., 0::2] = xp[None, :, None] * fw
    ang[..., 1::2] = yp[:, None, None] * fh
    ang = ang.reshape(hs * ws, head_dim // 2)
    return ang.cos().float(), ang.sin().float()


def rope_1d_text(head_dim: int, length: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    f = 1.0 / theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim)
    ang = torch.arange(length, dtype=torch.float64)[:, None] * f
    return ang.cos().float(), ang.sin().float()


def sincos_2d_pos(dim: int, h: int, w: int) -> torch.Tensor:
    """[h * w, dim]: first half from the column, second half from the row, each (sin | cos) over dim / 4 frequencies;
    axes longer than the training maximum are compressed onto it (PID_PIXEL_POS_ABS=1 keeps absolute positions)."""
    d = dim // 2
    half = d // 2
    omega = 1.0 / 10000.0 ** (torch.arange(half, dtype=torch.float64) / (d / 2.0))
    absolute = os.environ.get("PID_PIXEL_POS_ABS") == "1"
    sc = lambda n: 1.0 if absolute or n <= PIXEL_POS_TRAIN_MAX else PIXEL_POS_TRAIN_MAX / n                     # noqa: E731
    one = lambda pos: torch.cat([(pos[:, None] * omega).sin(), (pos[:, None] * omega).cos()], dim=1)             # noqa: E731
    ex = one(torch.arange(w, dtype=torch.float64) * sc(w))
    ey = one(torch.arange(h, dtype=torch.float64) * sc(h))
    return torch.cat([ex[None].expand(h, w, d), ey[:, None].expand(h, w, d)], dim=-1).reshape(h * w, dim).float()


def unfold_patches(x: torch.Tensor, p: int) -> torch.Tensor:
    B, C, H, W = x.shape
    return x.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)


def fold_patches(x: torch.Tensor, c: int, hs: int, ws: int, p: int) -> torch.Tensor:
    return x.reshape(x.shape[0], c, p, p, hs, ws).permute(0, 1, 4, 2, 5, 3).reshape(x.shape[0], c, hs * p, ws * p)


# ---- network ----------------------------------------------------------------------------------------------------------------
def _mod(x, w, scale, shift):
    return (nd.rms_norm(x, w, RMS_EPS).float() * (1.0 + scale.float()) + shift.float()).to(x.dtype)


def _heads(t: torch.Tensor, heads: int):
    B, S, _ = t.shape
    q, k, v = t.view(B, S, 3, heads, -1).unbind(2)
    return q, k, v


class PidNet:
    """PixDiT with the low-quality-latent adapter. forward(x, t, y, lq_latent, sigma) -> velocity in pixel space."""

    def __init__(self, weights: dict[str, torch.Tensor], cfg: PidConfig, device="cpu", prefix: str = ""):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        conv = ("lq_proj.latent_proj.",)
        self.w = nd.WeightBag({k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}, self.dtype, self.device,
                              keep_fp32=conv + ("log_alpha",))
        need = ["s_embedder.proj.weight", "y_pos_embedding", "final_layer.linear.weight", "lq_proj.latent_proj.0.weight"]
        for k in need:
            if k not in self.w:
                raise LoadError(f"pid: checkpoint lacks {k}")
        proj_in = self.w["lq_proj.latent_proj.0.weight"].shape[1]
        self.unpatchify = self._unpatchify_factor(cfg.lq_latent_channels, proj_in)
        self.upsample = max((cfg.sr_scale * cfg.latent_spatial_down_factor) // (cfg.patch_size * self.unpatchify), 1)

    @staticmethod
    def _unpatchify_factor(latent_channels: int, proj_in: int) -> int:
        if proj_in == latent_channels:
            return 1
        if proj_in <= 0 or latent_channels % proj_in:
            raise LoadError(f"pid: latent channels ({latent_channels}) not a square multiple of the adapter's input ({proj_in})")
        f = int(round(math.sqrt(latent_channels // proj_in)))
        if f * f != latent_channels // proj_in:
            raise LoadError(f"pid: un-patchify ratio {latent_channels // proj_in} is not a perfect square")
        return f

    # -- adapter --
    def _conv(self, x, p):
        w, b = self.w[p + ".weight"], self.w.get(p + ".bias")
        if self.cfg.lq_replicate_padding:
            return F.conv2d(F.pad(x, (1, 1, 1, 1), mode="replicate"), w, b)
        return F.conv2d(x, w, b, padding=1)

    def _gn(self, x, p):
        return F.group_norm(x, GN_GROUPS, self.w[p + ".weight"].float(), self.w[p + ".bias"].float(), GN_EPS)

    def lq_features(self, lq: torch.Tensor) -> tuple[list[torch.Tensor], torch.Tensor | None]:
        """latent [B, C, zh, zw] -> (one [B, patches, hidden] feature per gated block, the pixel-stage feature or None).
        The trunk runs in fp32 through the framework's convolution: it is evaluated once per network call on a map of one
        cell per patch."""
        cfg, p = self.cfg, "lq_proj.latent_proj"
        x = lq.float().to(self.device)
        if self.unpatchify > 1:
            B, C, H, W = x.shape
            f = self.unpatchify
            x = x.reshape(B, C // (f * f), f, f, H, W).permute(0, 1, 4, 2, 5, 3).reshape(B, C // (f * f), H * f, W * f)
        if self.upsample > 1:
            x = F.interpolate(x, scale_factor=self.upsample, mode="nearest")
        x = self._conv(F.silu(self._conv(x, p + ".0")), p + ".2")
        for i in range(cfg.lq_num_res_blocks):
            r = f"{p}.{i + 3}.block"
            h = self._conv(F.silu(self._gn(x, r + ".0")), r + ".2")
            x = x + self._conv(F.silu(self._gn(h, r + ".3")), r + ".5")
        tokens = x.permute(0, 2, 3, 1).reshape(x.shape[0], -1, x.shape[1]).to(self.dtype)
        feats = [self.w.lin(tokens, f"lq_proj.output_heads.{i}") for i in range(cfg.num_lq_outputs)]
        pit = self.w.lin(tokens, "lq_proj.pit_head") if cfg.pit_lq_inject else None
        return feats, pit

    def _gate(self, p: str, x, lq, sigma):
        """x + sigmoid(W [x | lq] - sigma * exp(log_alpha)) * lq: the noisier the latent, the less of it is let in."""
        logit = self.w.lin(torch.cat([x, lq], dim=-1), p + ".content_proj").float()
        off = sigma.float().view(-1, 1, 1) * self.w[p + ".log_alpha"].float().exp()
        return (x.float() + torch.sigmoid(logit - off) * lq.float()).to(x.dtype)

    # -- attention --
    def _joint_attention(self, p, x, y, rope_img, rope_txt):
        w, H = self.w, self.cfg.num_groups
        qx, kx, vx = _heads(w.lin(x, p + ".qkv_x"), H)
        qy, ky, vy = _heads(w.lin(y, p + ".qkv_y"), H)
        qx, kx = nd.rms_norm(qx, w[p + ".q_norm_x.weight"], RMS_EPS), nd.rms_norm(kx, w[p + ".k_norm_x.weight"], RMS_EPS)
        qy, ky = nd.rms_norm(qy, w[p + ".q_norm_y.weight"], RMS_EPS), nd.rms_norm(ky, w[p + ".k_norm_y.weight"], RMS_EPS)
        qx, kx = nd.rope_interleaved(qx, *rope_img), nd.rope_interleaved(kx, *rope_img)
        qy, ky = nd.rope_interleaved(qy, *rope_txt), nd.rope_interleaved(ky, *rope_txt)
        o = nd.attention(torch.cat([qy, qx], 1), torch.cat([ky, kx], 1), torch.cat([vy, vx], 1))
        ny = y.shape[1]
        return w.lin(o[:, ny:], p + ".proj_x"), w.lin(o[:, :ny], p + ".proj_y")

    def _ffn(self, p, x):
        w = self.w
        return w.lin(w.lin(x, p + ".w1", act="silu") * w.lin(x, p + ".w3"), p + ".w2")

    @torch.no_grad()
    def forward(self, x: torch.Tensor, t: torch.Tensor, y: torch.Tensor, lq_latent: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
        """x [B, 3, H, W] noisy pixels, t [B] (student time * 1000), y [B, L, txt dim] caption states, lq_latent the generator's
        latent (normalised for its latent space), sigma [B] how noisy that latent still is."""
        cfg, w = self.cfg, self.w
        P = cfg.patch_size
        B, _, Hh, Ww = x.shape
        hs, ws = Hh // P, Ww // P
        L = hs * ws
        dev = self.device
        feats, pit = self.lq_features(lq_latent)
        x = x.to(dev)
        temb = nd.sinusoidal_embedding(t.to(dev).float(), 256, max_period=10.0).to(self.dtype)
        temb = w.lin(w.lin(temb, "t_embedder.mlp.0", act="silu"), "t_embedder.mlp.2").view(B, 1, cfg.hidden_size)
        ltxt = min(y.shape[1], cfg.txt_max_length)
        yv = w.lin(y[:, :ltxt].to(dev, self.dtype), "y_embedder.proj")
        if "y_embedder.norm.weight" in w:
            yv = nd.rms_norm(yv, w["y_embedder.norm.weight"], RMS_EPS)
        yv = yv + w["y_pos_embedding"][:, :ltxt]
        cond = F.silu(temb.float()).to(self.dtype)
        rope_img = tuple(r.to(dev) for r in rope_2d_ntk(cfg.head_dim, hs, ws, cfg.rope_ref_h // P, cfg.rope_ref_w // P))
        rope_txt = tuple(r.to(dev) for r in rope_1d_text(cfg.head_dim, ltxt, cfg.text_rope_theta))
        s = w.lin(unfold_patches(x.to(self.dtype), P), "s_embedder.proj")
        if "s_embedder.norm.weight" in w:
            s = nd.rms_norm(s, w["s_embedder.norm.weight"], RMS_EPS)
        sig = sigma.to(dev)
        for i in range(cfg.patch_depth):
            if cfg.lq_interval <= 1 or i % cfg.lq_interval == 0:
                k = i // cfg.lq_interval if cfg.lq_interval > 1 else i
                if k < len(feats):
                    s = self._gate(f"lq_proj.gate_modules.{k}", s, feats[k], sig)
            b = f"patch_blocks.{i}"
            mx = w.lin(cond, b + ".adaLN_modulation_img.0").chunk(6, dim=-1)
            my = w.lin(cond, b + ".adaLN_modulation_txt.0").chunk(6, dim=-1)
            ax, ay = self._joint_attention(b + ".attn", _mod(s, w[b + ".norm_x1.weight"], mx[1], mx[0]),
                                           _mod(yv, w[b + ".norm_y1.weight"], my[1], my[0]), rope_img, rope_txt)
            s = (s.float() + ax.float() * mx[2].float()).to(self.dtype)
            yv = (yv.float() + ay.float() * my[2].float()).to(self.dtype)
            s = (s.float() + self._ffn(b + ".mlp_x", _mod(s, w[b + ".norm_x2.weight"], mx[4], mx[3])).float() * mx[5].float()).to(self.dtype)
            yv = (yv.float() + self._ffn(b + ".mlp_y", _mod(yv, w[b + ".norm_y2.weight"], my[4], my[3])).float() * my[5].float()).to(self.dtype)
        s = F.silu(s.float() + temb.float()).to(self.dtype)
        if cfg.pit_lq_inject and pit is not None:
            s = self._gate("pit_lq_gate", s, pit, sig)
        s_cond = s.reshape(B * L, cfg.hidden_size)
        # pixel stage: every pixel of a patch is a token of width pixel_hidden_size, modulated by its patch's state
        pd, p2 = cfg.pixel_hidden_size, P * P
        xp = w.lin(x.permute(0, 2, 3, 1).to(self.dtype), "pixel_embedder.proj") + sincos_2d_pos(pd, Hh, Ww).to(dev, self.dtype).view(1, Hh, Ww, pd)
        xp = xp.reshape(B, hs, P, ws, P, pd).permute(0, 1, 3, 2, 4, 5).reshape(B * L, p2, pd)
        rope_pix = tuple(r.to(dev) for r in rope_2d_ntk(cfg.pixel_head_dim, hs, ws, cfg.rope_ref_h // P, cfg.rope_ref_w // P))
        for i in range(cfg.pixel_depth):
            b = f"pixel_blocks.{i}"
            m = w.lin(s_cond, b + ".adaLN_modulation.0").view(B * L, p2, 6 * pd).chunk(6, dim=-1)
            h = _mod(xp, w[b + ".norm1.weight"], m[1], m[0]).reshape(B * L, p2 * pd)
            hc = w.lin(h, b + ".compress_to_attn").view(B, L, cfg.pixel_attn_hidden_size)
            q, k, v = _heads(w.lin(hc, b + ".attn.qkv"), cfg.pixel_num_groups)
            q, k = nd.rms_norm(q, w[b + ".attn.q_norm.weight"], RMS_EPS), nd.rms_norm(k, w[b + ".attn.k_norm.weight"], RMS_EPS)
            a = w.lin(nd.attention(nd.rope_interleaved(q, *rope_pix), nd.rope_interleaved(k, *rope_pix), v), b + ".attn.proj")
            a = w.lin(a.reshape(B * L, -1), b + ".expand_from_attn").view(B * L, p2, pd)
            xp = (xp.float() + a.float() * m[2].float()).to(self.dtype)
            h = _mod(xp, w[b + ".norm2.weight"], m[4], m[3])
            h = w.lin(w.lin(h, b + ".mlp.fc1", act="gelu"), b + ".mlp.fc2")
            xp = (xp.float() + h.float() * m[5].float()).to(self.dtype)
        out = w.lin(nd.rms_norm(xp, w["final_layer.norm.weight"], RMS_EPS), "final_layer.linear").float()
        out = out.reshape(B, L, p2, cfg.in_channels).permute(0, 3, 2, 1)
        return fold_patches(out, cfg.in_channels, hs, ws, P)


# ---- tiling -----------------------------------------------------------------------------------------------------------------
def tile_axis(n: int, tile: int, overlap: int) -> list[tuple[int, int]]:
    """Full-size windows covering [0, n): strided by tile - overlap, the last one pulled back to end at n."""
    if n <= tile:
        return [(0, n)]
    stride, out, s = max(tile - overlap, 1), [], 0
    while True:
        e = min(s + tile, n)
        win = (max(e - tile, 0), e)
        if not out or out[-1] != win:
            out.append(win)
        if e >= n:
            return out
        s += stride


def plan_tiles(h: int, w: int, tile: int, overlap: int, align: int) -> list[tuple[int, int, int, int]]:
    align = max(align, 1)
    tile = max(tile // align * align, align)
    overlap = min(max(overlap // align * align, 0), tile - align)
    return [(y0, y1, x0, x1) for y0, y1 in tile_axis(h, tile, overlap) for x0, x1 in tile_axis(w, tile, overlap)]


def axis_ramp(n: int, fade_start: bool, fade_end: bool, overlap: int) -> torch.Tensor:
    ov = max(overlap, 1)
    i = torch.arange(n, dtype=torch.float32)
    w = torch.ones(n)
    if fade_start:
        w = torch.where(i < ov, torch.minimum(w, (i + 1.0) / (ov + 1.0)), w)
    if fade_end:
        w = torch.where(i >= n - ov, torch.minimum(w, (n - i) / (ov + 1.0)), w)
    return w.clamp(min=1e-4)


def forward_tiled(net: PidNet, x, t, y, lq, sigma, tile: int, overlap: int) -> torch.Tensor:
    """One network evaluation as overlapping tiles (aligned to the pixels of one latent cell), blended with ramps that fade
    only at interior tile edges."""
    H, W = x.shape[2:]
    f = max(H // lq.shape[2], 1)
    plan = plan_tiles(H, W, tile, overlap, f)
    if len(plan) == 1:
        return net.forward(x, t, y, lq, sigma)
    acc = torch.zeros(x.shape[0], 3, H, W)
    wsum = torch.zeros(1, 1, H, W)
    for y0, y1, x0, x1 in plan:
        v = net.forward(x[:, :, y0:y1, x0:x1], t, y, lq[:, :, y0 // f:y1 // f, x0 // f:x1 // f], sigma).float().cpu()
        wt = axis_ramp(y1 - y0, y0 > 0, y1 < H, overlap)[:, None] * axis_ramp(x1 - x0, x0 > 0, x1 < W, overlap)[None, :]
        acc[:, :, y0:y1, x0:x1] += v * wt
        wsum[:, :, y0:y1, x0:x1] += wt
    return acc / wsum


# ---- memory planning --------------------------------------------------------------------------------------------------------
GIB = 1024.0 ** 3


def resident_full_gib(b: float, th: float, tw: float) -> float:
    return 6.0 * b * 3.0 * th * tw * 4.0 / GIB                  # noise, eps draws, x, x0, accumulators at output resolution


def forward_activations_gib(b: float, fh: float, fw: float, patch: int, hidden: int) -> float:
    return (3.0 * b * 3.0 * fh * fw * 4.0 + 8.0 * b * (fh / patch) * (fw / patch) * hidden * 4.0) / GIB


def estimated_decode_peak_gib(b, th, tw, patch, hidden) -> float:
    return resident_full_gib(b, th, tw) + forward_activations_gib(b, th, tw, patch, hidden)


def tiled_peak_gib(b, th, tw, tile, patch, hidden) -> float:
    return resident_full_gib(b, th, tw) + forward_activations_gib(b, min(tile, th), min(tile, tw), patch, hidden)


def plan_tile_edge(b, th, tw, patch, hidden, safe_gib: float) -> tuple[int, int, bool]:
    """(tile edge, overlap, whole output fits): the largest aligned edge whose forward activations fit beside the resident
    buffers, at most the preferred edge, at least the minimum edge."""
    out_edge = max(th, tw)
    if estimated_decode_peak_gib(b, th, tw, patch, hidden) <= safe_gib:
        return out_edge, DEFAULT_TILE_OVERLAP, True
    avail = max(safe_gib - resident_full_gib(b, th, tw), 0.0)
    per = forward_activations_gib(b, 1.0, 1.0, patch, hidden)
    mem_edge = int(math.sqrt(max(avail / per, 0.0))) if per > 0 else out_edge
    edge = max(max(min(mem_edge, PREFERRED_TILE_EDGE, out_edge), MIN_TILE_EDGE) // TILE_ALIGN * TILE_ALIGN, TILE_ALIGN)
    return edge, DEFAULT_TILE_OVERLAP, False


def guard(model_id: str, count: int, width: int, height: int, scale: int, cfg: PidConfig, safe_gib: float) -> None:
    tw, th, b = width * scale, height * scale, max(count, 1)
    floor = tiled_peak_gib(b, th, tw, MIN_TILE_EDGE, cfg.patch_size, cfg.hidden_size)
    if floor > safe_gib:
        raise InferenceError(f"{model_id}: a PiD decode at {tw}x{th} (super-resolved {scale}x from {width}x{height}) needs about "
                             f"{floor:.0f} GB even tiled at the minimum {MIN_TILE_EDGE}px tile, above the {safe_gib:.0f} GB budget; "
                             "reduce the resolution or disable PiD for this request")


# ---- sampler ----------------------------------------------------------------------------------------------------------------
class Sampler:
    def __init__(self, t_list=STUDENT_T_LIST, timescale: float = FM_TIMESCALE, sde: bool = True):
        self.t_list, self.timescale, self.sde = list(t_list), timescale, sde

    @property
    def steps(self) -> int:
        return max(len(self.t_list) - 1, 0)

    @property
    def num_eps(self) -> int:
        return sum(1 for t in self.t_list[1:] if t > 0.0) if self.sde else 0

    def run(self, forward, noise: torch.Tensor, eps: list[torch.Tensor], cancel=lambda: False) -> torch.Tensor:
        """forward(x, t_scaled [B]) -> velocity. SDE: each step predicts the clean image x - t v and re-noises it to the next
        time with a fresh draw; the last step returns the prediction. ODE: Euler on the velocity. Output clamped to [-1, 1]."""
        x, ei, B = noise, 0, noise.shape[0]
        for i in range(self.steps):
            if cancel():
                raise Canceled("pid: cancelled")
            t_cur, t_next = self.t_list[i], self.t_list[i + 1]
            v = forward(x, torch.full((B,), t_cur * self.timescale)).float().cpu()
            if t_next > 0.0:
                if self.sde:
                    x = (x - v * t_cur) * (1.0 - t_next) + eps[ei] * t_next
                    ei += 1
                else:
                    x = x + v * (t_next - t_cur)
            else:
                x = x - v * t_cur
        return x.clamp(-1.0, 1.0)

    def draws(self, seed: int, b: int, h: int, w: int) -> tuple[torch.Tensor, list[torch.Tensor]]:
        from .seed import seeded_normal

        flat = seeded_normal(seed, (1 + self.num_eps) * b * 3 * h * w).view(1 + self.num_eps, b, 3, h, w)
        return flat[0], [flat[i + 1] for i in range(self.num_eps)]


# ---- caption ----------------------------------------------------------------------------------------------------------------
def select_index(max_len: int) -> list[int]:
    return [0] + list(range(max_len - (MODEL_MAX_LENGTH - 1), max_len))


class CaptionEncoder:
    """Gemma-2 states of (instruction prefix + caption): padded to prefix length + 298 tokens, padding masked as keys,
    final norm applied; kept are position 0 and the last 299 positions."""

    def __init__(self, gemma_dir: Path, device="cpu", chi_prompt: str | None = None):
        import json

        from ..contracts.gen_core.tokenizer import TextTokenizer, TokenizerConfig
        from ..io.safetensors_io import load_dir, load_file
        from ..models.config import ModelConfig
        from ..models.oracle import OracleLlama

        gemma_dir, self.device = Path(gemma_dir), torch.device(device)
        tk, cj = gemma_dir / "tokenizer.json", gemma_dir / "config.json"
        if not tk.is_file() or not cj.is_file():
            raise LoadError(f"pid gemma encoder: {gemma_dir} lacks tokenizer.json or config.json")
        merged = gemma_dir / GEMMA_MERGED_FILE
        w = load_file(merged) if merged.is_file() else load_dir(gemma_dir)
        cfg = ModelConfig.from_json(json.loads(cj.read_text(encoding="utf-8")))
        dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.lm = OracleLlama(cfg, w, dt, self.device)
        self.tok = TextTokenizer.from_file(tk, TokenizerConfig(max_length=4096))
        self.chi_prompt = chi_prompt if chi_prompt is not None else CHI_PROMPT
        self.num_chi_tokens = len(self.tok.encode_ids(self.chi_prompt, True))

    def token_ids(self, caption: str) -> tuple[list[int], int]:
        max_len = self.num_chi_tokens + MODEL_MAX_LENGTH - 2
        ids = self.tok.encode_ids(self.chi_prompt + caption, True)[:max_len]
        return ids + [PAD_ID] * (max_len - len(ids)), len(ids)

    @torch.no_grad()
    def encode(self, caption: str) -> torch.Tensor:
        ids, real = self.token_ids(caption)
        n = len(ids)
        i = torch.arange(n, device=self.device)
        mask = torch.zeros(n, n, device=self.device)
        mask = mask.masked_fill(i[None, :] > i[:, None], -1e9).masked_fill((i >= real)[None, :], -1e9)
        t = torch.tensor([ids], dtype=torch.int64, device=self.device)
        h = self.lm._norm(self.lm.hidden_states(t, None, additive_mask=mask[None, None].to(self.lm.dtype)), "model.norm.weight")
        return h[:, select_index(n)].float()


# ---- engine -----------------------------------------------------------------------------------------------------------------
def flow_capture_for_request(use_pid: bool, capture_sigma: float | None, sigmas: list[float], start_step: int) -> tuple[float, int]:
    """(sigma at which the latent is handed to PiD, number of schedule entries to keep). Without PiD, or when the capture
    point falls inside the steps a reference image already skipped, the whole schedule runs and the latent is clean."""
    from ..contracts.gen_core.sampling.policy import flow_capture_plan

    plan = flow_capture_plan(sigmas, capture_sigma) if use_pid else None
    if plan is not None and plan[0] > start_step + 1:
        return plan[1], plan[0]
    return 0.0, len(sigmas)


class PidDecoder:
    """One generation's decoder: bound to its caption states, the latent's remaining noise level and the seed."""

    def __init__(self, net: PidNet, sampler: Sampler, caption: torch.Tensor, sigma: float, seed: int, cancel=lambda: False,
                 tile: tuple[int, int] | None = None):
        self.net, self.sampler, self.caption, self.sigma, self.seed, self.cancel, self.tile = net, sampler, caption, sigma, seed, cancel, tile

    def target_hw(self, latents: torch.Tensor) -> tuple[int, int]:
        f = self.net.cfg.latent_spatial_down_factor * self.net.cfg.sr_scale
        return latents.shape[2] * f, latents.shape[3] * f

    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """latents [B, C, zh, zw] (the generator's latent, as its sampler leaves it) -> image [B, 3, zh * f, zw * f] in
        [-1, 1]. The registry's per-space normalisation describes the space the student was trained on."""
        B = latents.shape[0]
        th, tw = self.target_hw(latents)
        sig = torch.full((B,), float(self.sigma))
        noise, eps = self.sampler.draws(self.seed, B, th, tw)
        lat = latents.float()
        if self.tile is not None and (th > self.tile[0] or tw > self.tile[0]):
            fwd = lambda x, t: forward_tiled(self.net, x, t, self.caption, lat, sig, *self.tile)            # noqa: E731
        else:
            fwd = lambda x, t: self.net.forward(x, t, self.caption, lat, sig)                               # noqa: E731
        return self.sampler.run(fwd, noise, eps, self.cancel)


class PidEngine:
    """Loaded once per (checkpoint, latent space); `decoder(caption, sigma, seed)` mints a per-generation decoder."""

    def __init__(self, weights: dict[str, torch.Tensor], spec: BackboneSpec, caption: CaptionEncoder, device="cpu",
                 base_cfg: PidConfig | None = None):
        self.spec, self.caption, self.device = spec, caption, torch.device(device)
        self.cfg = config_for_spec(spec, detect_v1pt5(weights), base_cfg)
        self.net = PidNet(weights, self.cfg, device)
        self.sampler = Sampler()

    @staticmethod
    def load(checkpoint: Path, gemma_dir: Path, backbone: str, backend: str = "b200", base_cfg: PidConfig | None = None) -> "PidEngine":
        from ..io.safetensors_io import load_file

        spec = lookup(backbone)
        if spec is None:
            raise LoadError(f"pid: unknown / out-of-scope backbone {backbone!r} (no PiD latent-space mapping)")
        if not Path(checkpoint).is_file():
            raise LoadError(f"pid checkpoint: expected the converted .safetensors file, got {checkpoint}")
        dev = "cuda" if backend == "b200" else "cpu"
        return PidEngine(load_file(checkpoint), spec, CaptionEncoder(gemma_dir, dev), dev, base_cfg)

    @property
    def scale(self) -> int:
        return self.cfg.sr_scale

    @property
    def vae_compression(self) -> int:
        return self.cfg.latent_spatial_down_factor

    def decoder(self, caption: str, sigma: float, seed: int, cancel=lambda: False, safe_gib: float | None = None,
                batch: int = 1, latent_hw: tuple[int, int] | None = None) -> PidDecoder:
        tile = None
        if latent_hw is not None:
            if safe_gib is None:
                safe_gib = float(os.environ.get("PID_DECODE_BUDGET_GIB", "120"))
            f = self.vae_compression * self.scale
            edge, overlap, whole = plan_tile_edge(batch, latent_hw[0] * f, latent_hw[1] * f, self.cfg.patch_size, self.cfg.hidden_size, safe_gib)
            tile = None if whole else (edge, overlap)
        return PidDecoder(self.net, self.sampler, self.caption.encode(caption), sigma, seed, cancel, tile)


def resolve_pid_decoder(engine: "PidEngine | None", req, base_seed: int, model_id: str, capture_sigma: float = 0.0,
                        capture_wired: bool = False, safe_gib: float | None = None) -> "PidDecoder | None":
    """The request's decoder, or None when it did not ask for PiD. Asking without a loaded engine is an error; so is an
    early-stop capture on a latent space whose generator does not hand over noisy latents (`capture_wired`). The output
    is `scale` times the requested size, so the memory guard and the tile plan are sized for that."""
    if not req.use_pid:
        return None
    safe_gib = check_pid_request(engine, req, model_id, capture_wired, safe_gib)
    f = engine.vae_compression
    return engine.decoder(req.prompt, capture_sigma, base_seed, req.cancel.is_cancelled, safe_gib, max(req.count, 1),
                          (req.height // f, req.width // f))


def check_pid_request(engine: "PidEngine | None", req, model_id: str, capture_wired: bool = False,
                      safe_gib: float | None = None) -> float:
    """The refusals of a request that asks for PiD, before any work is done -> the memory budget in GiB."""
    if req.pid_capture_sigma is not None and not capture_wired:
        raise InferenceError(f"{model_id}: pid_capture_sigma (early stop on a noisy latent) is not wired for this latent space")
    if engine is None:
        raise InferenceError(f"{model_id}: use_pid was requested but no PiD decoder is loaded (load with LoadSpec.pid)")
    if safe_gib is None:
        safe_gib = float(os.environ.get("PID_DECODE_BUDGET_GIB", "0")) or _device_budget_gib(engine.device)
    guard(model_id, req.count, req.width, req.height, engine.scale, engine.cfg, safe_gib)
    return safe_gib


def _device_budget_gib(device: torch.device) -> float:
    """0.85 of the device's memory; 16 GiB on a host without one."""
    if device.type == "cuda":
        return torch.cuda.get_device_properties(device).total_memory * 0.85 / GIB
    return 16.0


# ---- synthetic checkpoint ---------------------------------------------------------------------------------------------------
def random_pid_weights(cfg: PidConfig, seed: int = 0, proj_in: int | None = None) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)                      # noqa: E731
    w: dict[str, torch.Tensor] = {}
    H, pd, pa, p2 = cfg.hidden_size, cfg.pixel_hidden_size, cfg.pixel_attn_hidden_size, cfg.patch_size ** 2

    def lin(p, o, i, bias=True, std=None):
        w[p + ".weight"] = rn(o, i) * (std if std is not None else 1.0 / math.sqrt(i))
        if bias:
            w[p + ".bias"] = rn(o) * 0.02

    norm = lambda p, d: w.__setitem__(p + ".weight", 1 + 0.05 * rn(d))             # noqa: E731
    lin("s_embedder.proj", H, 3 * p2)
    norm("s_embedder.norm", H)
    lin("y_embedder.proj", H, cfg.txt_embed_dim)
    norm("y_embedder.norm", H)
    w["y_pos_embedding"] = rn(1, cfg.txt_max_length, H) * 0.05
    lin("t_embedder.mlp.0", H, 256)
    lin("t_embedder.mlp.2", H, H)
    lin("pixel_embedder.proj", pd, 3)
    for i in range(cfg.patch_depth):
        b = f"patch_blocks.{i}"
        for n in ("norm_x1", "norm_y1", "norm_x2", "norm_y2"):
            norm(f"{b}.{n}", H)
        for s in "xy":
            lin(f"{b}.attn.qkv_{s}", 3 * H, H)
            lin(f"{b}.attn.proj_{s}", H, H)
            norm(f"{b}.attn.q_norm_{s}", cfg.head_dim)
            norm(f"{b}.attn.k_norm_{s}", cfg.head_dim)
            for n, o, ii in (("w1", 2 * H, H), ("w3", 2 * H, H), ("w2", H, 2 * H)):
                lin(f"{b}.mlp_{s}.{n}", o, ii, bias=False)
        lin(b + ".adaLN_modulation_img.0", 6 * H, H, std=0.02)
        lin(b + ".adaLN_modulation_txt.0", 6 * H, H, std=0.02)
    for i in range(cfg.pixel_depth):
        b = f"pixel_blocks.{i}"
        lin(b + ".compress_to_attn", pa, p2 * pd)
        lin(b + ".expand_from_attn", p2 * pd, pa)
        norm(b + ".norm1", pd)
        norm(b + ".norm2", pd)
        lin(b + ".attn.qkv", 3 * pa, pa)
        lin(b + ".attn.proj", pa, pa)
        norm(b + ".attn.q_norm", cfg.pixel_head_dim)
        norm(b + ".attn.k_norm", cfg.pixel_head_dim)
        lin(b + ".mlp.fc1", 4 * pd, pd)
        lin(b + ".mlp.fc2", pd, 4 * pd)
        lin(b + ".adaLN_modulation.0", p2 * 6 * pd, H, std=0.02)
    norm("final_layer.norm", pd)
    lin("final_layer.linear", cfg.in_channels, pd)
    hid, cin = cfg.lq_hidden_dim, proj_in if proj_in is not None else cfg.lq_latent_channels
    conv = lambda p, o, i: (w.__setitem__(p + ".weight", rn(o, i, 3, 3) / math.sqrt(9 * i)), w.__setitem__(p + ".bias", rn(o) * 0.02))   # noqa: E731
    conv("lq_proj.latent_proj.0", hid, cin)
    conv("lq_proj.latent_proj.2", hid, hid)
    for i in range(cfg.lq_num_res_blocks):
        r = f"lq_proj.latent_proj.{i + 3}.block"
        for n in (".0", ".3"):
            w[r + n + ".weight"], w[r + n + ".bias"] = 1 + 0.05 * rn(hid), 0.02 * rn(hid)
        conv(r + ".2", hid, hid)
        conv(r + ".5", hid, hid)
    gate_rows = 1 if cfg.pit_lq_inject else H
    for i in range(cfg.num_lq_outputs):
        lin(f"lq_proj.output_heads.{i}", H, hid)
        lin(f"lq_proj.gate_modules.{i}.content_proj", gate_rows, 2 * H)
        w[f"lq_proj.gate_modules.{i}.log_alpha"] = rn(1) * 0.1
    if cfg.pit_lq_inject:
        lin("lq_proj.pit_head", H, hid)
        lin("pit_lq_gate.content_proj", 1, 2 * H)
        w["pit_lq_gate.log_alpha"] = rn(1) * 0.1
    return w
