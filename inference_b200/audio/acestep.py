"""ACE-Step 1.5 text-to-music (`acestep_v15_turbo`): style prompt + lyrics -> 48 kHz stereo, plus region edits and covers.

Behaviour follows the reference's candle-audio-acestep crate:
  - config.rs:10-330    the five component configs of a diffusers snapshot and their cross-checks
  - text.rs:20-75       prompt assembly (style text + bpm / key / time signature / language) and the token caps
  - condition.rs:60-287 the condition encoder: text projector, lyric encoder, timbre encoder on its learned token,
                        and the stored silence latent that stands in for "no source audio"
  - dit.rs:36-480       the AdaLN-Zero DiT: patch convolution over (source latents, mask, noisy latents), grouped-query
                        self-attention with per-head RMSNorm, half-split rotary phases and a symmetric sliding window
                        on alternate layers, ungated cross-attention, SwiGLU MLP, transposed-convolution un-patching
  - scheduler.rs:10-50  the shifted flow-match ladder and its Euler step
  - vae.rs:10-340       the Oobleck autoencoder (snake activations, weight-normed convolutions), decoder and encoder
  - tokenizer.rs:20-400 the cover path's attention pooler + finite scalar quantiser and its de-tokeniser
  - pipeline.rs:60-760  synthesize / edit (inpaint, repaint, extend) / cover, stitching with a bounded crossfade
  - model.rs:14-430     descriptor, request validation, the `sft_cover` component

One implementation serves both backends through `models.nn_dual`: on the device every projection is the tcgen05 GEMM,
full-attention layers run on the tcgen05 attention kernel, norms on the vectorised norm kernel; the oracle backend is
the same code in fp32.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, GenerationOutput, GenerationRequest, Generator,
                                            Modality, ModelDescriptor)
from ..contracts.gen_core.license import WeightLicense
from ..contracts.gen_core.media import AudioTrack
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec, ProgressDecoding, ProgressStep
from ..models import nn_dual as nd

MODEL_ID = "acestep_v15_turbo"
FAMILY = "acestep"
SAMPLE_RATE = 48_000
CHANNELS = 2
MAX_DURATION_SECS = 600.0
MAX_STEPS = 200
DEFAULT_SECONDS = 60.0
DEFAULT_STEPS = 8
COVER_STEPS = 24
DEFAULT_SHIFT = 3.0
MAX_TEXT_LEN = 256
MAX_LYRIC_LEN = 2048
FREQ_DIM = 256
LANGUAGES = ("en", "zh", "ja", "ko", "fr", "de", "es", "it", "pt", "ru")
EDIT_MODES = ("inpaint", "repaint", "extend", "cover")
COVER_COMPONENT = "sft_cover"
VAE_FILE = "diffusion_pytorch_model.safetensors"
FSQ_LEVELS = (8, 8, 8, 5, 5, 5)
MAX_CROSSFADE = 960                                   # 20 ms at 48 kHz

ACESTEP_LICENSE = WeightLicense("MIT", "MIT License", "https://huggingface.co/ACE-Step/acestep-v15-xl-turbo-diffusers",
                                "ACE-Step v1.5 XL Turbo (c) ACE-Step, licensed under MIT", True,
                                "Bundled text_encoder (Qwen3-Embedding-0.6B) is redistributed under Apache-2.0.")


# ---- text -------------------------------------------------------------------------------------------------------------------
@dataclass
class Metadata:
    bpm: float | None = None
    key: str | None = None
    time_signature: str | None = None
    vocal_language: str | None = None


def build_prompt(prompt: str, meta: Metadata) -> str:
    """Whitespace-collapsed style text followed by the present metadata fields, in a fixed order."""
    parts = []
    base = " ".join(prompt.split())
    if base:
        parts.append(base)
    if meta.bpm is not None:
        parts.append(f"bpm: {int(meta.bpm)}" if float(meta.bpm).is_integer() else f"bpm: {meta.bpm}")
    for label, value in (("key", meta.key), ("time signature", meta.time_signature), ("language", meta.vocal_language)):
        if value is not None and value.strip():
            parts.append(f"{label}: {value.strip()}")
    return ", ".join(parts)


# ---- schedule ---------------------------------------------------------------------------------------------------------------
def flow_sigmas(steps: int, shift: float) -> list[float]:
    """steps + 1 values: the linear ladder 1 - i / steps bent by `shift`, then the terminal 0."""
    steps = max(steps, 1)
    out = []
    for i in range(steps):
        s = 1.0 - i / steps
        out.append(s if abs(shift - 1.0) < 2.3e-16 else shift * s / (1.0 + (shift - 1.0) * s))
    return out + [0.0]


# ---- configs ----------------------------------------------------------------------------------------------------------------
@dataclass
class VaeConfig:
    audio_channels: int
    channel_multiples: list[int]
    decoder_channels: int
    decoder_input_channels: int
    downsampling_ratios: list[int]
    sampling_rate: int

    @property
    def hop_length(self) -> int:
        return math.prod(self.downsampling_ratios)

    @property
    def latents_per_second(self) -> float:
        return self.sampling_rate / self.hop_length

    def validate(self) -> None:
        if self.audio_channels != 2:
            raise LoadError(f"acestep VAE: audio_channels {self.audio_channels} unsupported (the autoencoder is stereo)")
        if len(self.channel_multiples) != len(self.downsampling_ratios):
            raise LoadError("acestep VAE: channel_multiples and downsampling_ratios differ in length")
        if self.hop_length == 0 or self.sampling_rate % self.hop_length:
            raise LoadError(f"acestep VAE: sampling_rate {self.sampling_rate} not divisible by hop_length {self.hop_length}")


@dataclass
class TransformerConfig:
    in_channels: int
    audio_acoustic_hidden_dim: int
    encoder_hidden_size: int
    hidden_size: int
    intermediate_size: int
    head_dim: int
    num_attention_heads: int
    num_key_value_heads: int
    num_hidden_layers: int
    patch_size: int
    layer_types: list[str]
    sliding_window: int
    rms_norm_eps: float
    rope_theta: float
    attention_bias: bool = False
    is_turbo: bool = False

    def validate(self, vae: VaeConfig) -> None:
        a = self.audio_acoustic_hidden_dim
        if a != vae.decoder_input_channels:
            raise LoadError(f"acestep: DiT audio_acoustic_hidden_dim {a} != VAE decoder_input_channels {vae.decoder_input_channels}")
        if self.in_channels != 3 * a:
            raise LoadError(f"acestep: DiT in_channels {self.in_channels} != 3 x audio_acoustic_hidden_dim {a}")
        if len(self.layer_types) != self.num_hidden_layers:
            raise LoadError("acestep: DiT layer_types does not list one entry per layer")
        for t in self.layer_types:
            if t not in ("sliding_attention", "full_attention"):
                raise LoadError(f"acestep: DiT unknown layer_type {t!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise LoadError("acestep: DiT heads not a multiple of kv heads")
        if self.head_dim % 2:
            raise LoadError("acestep: DiT head_dim must be even for the rotary phases")


@dataclass
class EncoderConfig:
    """The transformer-layer shape shared by the condition encoder, the audio tokenizer and its de-tokenizer."""
    hidden_size: int
    intermediate_size: int
    head_dim: int
    num_attention_heads: int
    num_key_value_heads: int
    rms_norm_eps: float
    rope_theta: float
    extra: dict = field(default_factory=dict)

    @staticmethod
    def from_json(j: dict) -> "EncoderConfig":
        names = ("hidden_size", "intermediate_size", "head_dim", "num_attention_heads", "num_key_value_heads",
                 "rms_norm_eps", "rope_theta")
        for n in names:
            if n not in j:
                raise LoadError(f"acestep: encoder config lacks {n}")
        cfg = EncoderConfig(**{n: j[n] for n in names}, extra={k: v for k, v in j.items() if k not in names})
        if cfg.num_attention_heads % cfg.num_key_value_heads:
            raise LoadError("acestep: encoder heads not a multiple of kv heads")
        return cfg


def _from_json(cls, j: dict, what: str):
    missing = [n for n, f in cls.__dataclass_fields__.items()
               if n not in j and f.default is f.default_factory]   # both MISSING: a required field
    if missing:
        raise LoadError(f"acestep: {what} config lacks {missing}")
    return cls(**{n: j[n] for n in cls.__dataclass_fields__ if n in j})


# ---- shared transformer layer -----------------------------------------------------------------------------------------------
def rope_tables(head_dim: int, length: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(length, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def _attend(w: nd.WeightBag, p: str, x: torch.Tensor, src: torch.Tensor, heads: int, kv_heads: int, hd: int, eps: float,
            rope=None, mask=None) -> torch.Tensor:
    """Grouped-query attention with per-head RMSNorm on q and k; `rope` = (cos, sin) rotates both (self-attention)."""
    B, S = x.shape[:2]
    L = src.shape[1]
    q = nd.rms_norm(w.lin(x, p + "to_q").view(B, S, heads, hd), w[p + "norm_q.weight"], eps)
    k = nd.rms_norm(w.lin(src, p + "to_k").view(B, L, kv_heads, hd), w[p + "norm_k.weight"], eps)
    v = w.lin(src, p + "to_v").view(B, L, kv_heads, hd)
    if rope is not None:
        q, k = nd.rope_half(q, *rope), nd.rope_half(k, *rope)
    return w.lin(nd.attention(q, k, v, mask=mask), p + "to_out.0")


def encoder_layer(w: nd.WeightBag, p: str, cfg: EncoderConfig, x: torch.Tensor) -> torch.Tensor:
    """Pre-norm layer: bidirectional rotary self-attention then SwiGLU, both plain residuals."""
    S = x.shape[1]
    rope = rope_tables(cfg.head_dim, S, cfg.rope_theta, x.device)
    h = nd.rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
    x = x + _attend(w, p + "self_attn.", h, h, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                    cfg.rms_norm_eps, rope)
    h = nd.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
    return x + w.lin(w.lin(h, p + "mlp.gate_proj", act="silu") * w.lin(h, p + "mlp.up_proj"), p + "mlp.down_proj")


def _stack(w: nd.WeightBag, p: str, cfg: EncoderConfig, x: torch.Tensor, layers: int) -> torch.Tensor:
    for i in range(layers):
        x = encoder_layer(w, f"{p}layers.{i}.", cfg, x)
    return nd.rms_norm(x, w[p + "norm.weight"], cfg.rms_norm_eps)


def _dtype_for(device: torch.device):
    return torch.bfloat16 if device.type == "cuda" else torch.float32


class ConditionEncoder:
    def __init__(self, cfg: EncoderConfig, weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = _dtype_for(self.device)
        for k in ("timbre_encoder.special_token", "silence_latent", "text_projector.weight"):
            if k not in weights:
                raise LoadError(f"acestep condition encoder: missing tensor {k!r}")
        self.w = nd.WeightBag(weights, self.dtype, self.device, keep_fp32=("silence_latent",))
        self.lyric_layers = int(cfg.extra["num_lyric_encoder_hidden_layers"])
        self.timbre_layers = int(cfg.extra["num_timbre_encoder_hidden_layers"])

    def src_latents(self, length: int) -> torch.Tensor:
        """[1, length, acoustic]: the stored silence latent, tiled when the request outlasts it."""
        s = self.w["silence_latent"]
        reps = -(-length // s.shape[1])
        return (s if reps == 1 else s.repeat(1, reps, 1))[:, :length].contiguous()

    @torch.no_grad()
    def encode(self, text_hidden: torch.Tensor, lyric_embeds: torch.Tensor | None) -> torch.Tensor:
        """[projected text | encoded lyrics | encoded timbre token] along the sequence."""
        w = self.w
        parts = [w.lin(text_hidden.to(self.dtype), "text_projector")]
        if lyric_embeds is not None:
            x = w.lin(lyric_embeds.to(self.dtype), "lyric_encoder.embed_tokens")
            parts.append(_stack(w, "lyric_encoder.", self.cfg, x, self.lyric_layers))
        parts.append(_stack(w, "timbre_encoder.", self.cfg, w["timbre_encoder.special_token"], self.timbre_layers))
        return torch.cat(parts, dim=1)


# ---- DiT --------------------------------------------------------------------------------------------------------------------
class AceStepDiT:
    def __init__(self, cfg: TransformerConfig, weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = _dtype_for(self.device)
        self.w = nd.WeightBag(weights, self.dtype, self.device)
        w = self.w
        # A stride-p convolution with a p-wide kernel is a projection of p stacked frames; the transposed one likewise.
        pi = w["proj_in_conv.weight"]                                          # [dim, in, p]
        self.w_in = pi.permute(0, 2, 1).reshape(pi.shape[0], -1).contiguous()  # columns ordered (tap, channel)
        po = w["proj_out_conv.weight"]                                         # [dim, acoustic, p]
        self.w_out = po.permute(2, 1, 0).reshape(-1, po.shape[0]).contiguous() # rows ordered (tap, channel)
        self.b_out = w["proj_out_conv.bias"].repeat(cfg.patch_size) if "proj_out_conv.bias" in w else None

    def embed_context(self, encoder_hidden: torch.Tensor) -> torch.Tensor:
        return self.w.lin(encoder_hidden.to(self.dtype), "condition_embedder")

    def _time(self, p: str, t: float) -> tuple[torch.Tensor, torch.Tensor]:
        w = self.w
        s = nd.sinusoidal_embedding(torch.tensor([t * 1000.0], device=self.device), FREQ_DIM).to(self.dtype)
        temb = w.lin(w.lin(s, p + "linear_1", act="silu"), p + "linear_2")
        return temb.float(), w.lin(F.silu(temb.float()).to(self.dtype), p + "time_proj").float()

    def sliding_mask(self, length: int) -> torch.Tensor:
        i = torch.arange(length, device=self.device)
        return (i[:, None] - i[None, :]).abs() <= self.cfg.sliding_window

    @torch.no_grad()
    def forward(self, hidden: torch.Tensor, context_latents: torch.Tensor, timestep: float, ctx: torch.Tensor,
                cancel=lambda: False) -> torch.Tensor | None:
        """hidden [1, T, acoustic] at `timestep` in [0, 1], context_latents [1, T, 2 * acoustic], ctx the embedded
        condition [1, S, dim] -> velocity [1, T, acoustic]; None when cancelled between blocks."""
        cfg, w = self.cfg, self.w
        H, KV, D, eps, p = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps, cfg.patch_size
        T = hidden.shape[1]
        x = torch.cat([context_latents, hidden], dim=-1).to(self.dtype)
        if T % p:
            x = F.pad(x, (0, 0, 0, p - T % p))
        N = x.shape[1] // p
        x = nd.linear(x.reshape(1, N, p * cfg.in_channels), self.w_in, w.get("proj_in_conv.bias"))
        temb_t, tp_t = self._time("time_embed.", timestep)
        temb_r, tp_r = self._time("time_embed_r.", 0.0)        # inference runs with r == t, so this branch sees 0
        temb, tproj = temb_t + temb_r, (tp_t + tp_r).view(1, 6, cfg.hidden_size)
        rope = rope_tables(D, N, cfg.rope_theta, self.device)
        window = self.sliding_mask(N) if "sliding_attention" in cfg.layer_types and N > cfg.sliding_window + 1 else None
        ctx = ctx.to(self.dtype)
        for i in range(cfg.num_hidden_layers):
            if cancel():
                return None
            b = f"layers.{i}."
            m = w[b + "scale_shift_table"].float() + tproj
            sh_a, sc_a, g_a, sh_f, sc_f, g_f = (m[:, j:j + 1] for j in range(6))
            h = (nd.rms_norm(x, w[b + "self_attn_norm.weight"], eps).float() * (1.0 + sc_a) + sh_a).to(self.dtype)
            mask = window if cfg.layer_types[i] == "sliding_attention" else None
            x = (x.float() + _attend(w, b + "self_attn.", h, h, H, KV, D, eps, rope, mask).float() * g_a).to(self.dtype)
            h = nd.rms_norm(x, w[b + "cross_attn_norm.weight"], eps)
            x = x + _attend(w, b + "cross_attn.", h, ctx, H, KV, D, eps)
            h = (nd.rms_norm(x, w[b + "mlp_norm.weight"], eps).float() * (1.0 + sc_f) + sh_f).to(self.dtype)
            f = w.lin(w.lin(h, b + "mlp.gate_proj", act="silu") * w.lin(h, b + "mlp.up_proj"), b + "mlp.down_proj")
            x = (x.float() + f.float() * g_f).to(self.dtype)
        m = w["scale_shift_table"].float() + temb[:, None]
        x = (nd.rms_norm(x, w["norm_out.weight"], eps).float() * (1.0 + m[:, 1:2]) + m[:, 0:1]).to(self.dtype)
        v = nd.linear(x, self.w_out, self.b_out).float().reshape(1, N * p, cfg.audio_acoustic_hidden_dim)
        return v[:, :T].contiguous()


# ---- Oobleck autoencoder ----------------------------------------------------------------------------------------------------
def fold_weight_norm(raw: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """weight = g * v / ||v|| (norm over all but the first axis), for both spellings of the parametrisation."""
    out = {}
    pairs = ((".weight_g", ".weight_v"), (".parametrizations.weight.original0", ".parametrizations.weight.original1"))
    for name, t in raw.items():
        for g_suf, v_suf in pairs:
            if name.endswith(g_suf):
                base = name[: -len(g_suf)]
                if base + v_suf not in raw:
                    raise LoadError(f"acestep VAE: {base} has a magnitude tensor without its direction tensor")
                v = raw[base + v_suf].float()
                norm = v.pow(2).sum(dim=tuple(range(1, v.dim())), keepdim=True).sqrt()
                out[base + ".weight"] = v * t.float() / norm
                break
            if name.endswith(v_suf):
                break
        else:
            out[name] = t.float()
    return out


def snake(x: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """x + sin^2(e^alpha x) / (e^beta + 1e-9), alpha / beta stored as logs, broadcast over [1, C, 1]."""
    return x + torch.sin(x * alpha.exp()).pow(2) / (beta.exp() + 1e-9)


class Oobleck:
    """Decoder (latents -> stereo waveform) and encoder (waveform -> posterior mean) of the audio autoencoder.
    Runs in fp32 on either device: the convolutions are framework calls, a small share of a generation."""

    def __init__(self, cfg: VaeConfig, weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        if not any(k.startswith("decoder.") for k in weights):
            raise LoadError("acestep VAE: no decoder.* tensors, not an Oobleck checkpoint")
        self.w = {k: v.to(self.device) for k, v in fold_weight_norm(weights).items()}
        self.has_encoder = any(k.startswith("encoder.") for k in self.w)

    def _get(self, k: str) -> torch.Tensor:
        if k not in self.w:
            raise LoadError(f"acestep VAE: missing tensor {k!r}")
        return self.w[k]

    def _snake(self, x, p):
        return snake(x, self._get(p + ".alpha"), self._get(p + ".beta"))

    def _conv(self, x, p, **kw):
        return F.conv1d(x, self._get(p + ".weight"), self.w.get(p + ".bias"), **kw)

    def _res(self, x, p, dilation):
        y = self._conv(self._snake(x, p + ".snake1"), p + ".conv1", padding=3 * dilation, dilation=dilation)
        y = self._conv(self._snake(y, p + ".snake2"), p + ".conv2")
        pad = (x.shape[-1] - y.shape[-1]) // 2
        return y + (x[..., pad: pad + y.shape[-1]] if pad > 0 else x)

    @torch.no_grad()
    def decode(self, z: torch.Tensor, cancel=lambda: False) -> torch.Tensor | None:
        """[1, latent, T] -> [1, 2, T * hop]."""
        x = self._conv(z.float(), "decoder.conv1", padding=3)
        for i, s in enumerate(reversed(self.cfg.downsampling_ratios)):
            if cancel():
                return None
            b = f"decoder.block.{i}"
            pad = -(-s // 2)
            x = F.conv_transpose1d(self._snake(x, b + ".snake1"), self._get(b + ".conv_t1.weight"),
                                   self.w.get(b + ".conv_t1.bias"), stride=s, padding=pad,
                                   output_padding=max(2 * s - (s + 2 * pad), 0))
            for j, d in enumerate((1, 3, 9)):
                x = self._res(x, f"{b}.res_unit{j + 1}", d)
        if cancel():
            return None
        return self._conv(self._snake(x, "decoder.snake1"), "decoder.conv2", padding=3)

    @torch.no_grad()
    def encode(self, wave: torch.Tensor, cancel=lambda: False) -> torch.Tensor | None:
        """[1, 2, frames] (a hop multiple) -> posterior mean [1, frames / hop, latent]."""
        if not self.has_encoder:
            raise LoadError("acestep VAE: the checkpoint has no encoder.* tensors (needed to edit or cover a source clip)")
        x = self._conv(wave.float(), "encoder.conv1", padding=3)
        for i, s in enumerate(self.cfg.downsampling_ratios):
            if cancel():
                return None
            b = f"encoder.block.{i}"
            for j, d in enumerate((1, 3, 9)):
                x = self._res(x, f"{b}.res_unit{j + 1}", d)
            x = self._conv(self._snake(x, b + ".snake1"), b + ".conv1", stride=s, padding=-(-s // 2))
        if cancel():
            return None
        params = self._conv(self._snake(x, "encoder.snake1"), "encoder.conv2", padding=1)
        return params[:, : self.cfg.decoder_input_channels].transpose(1, 2).contiguous()


# ---- cover: audio tokenizer / de-tokenizer ----------------------------------------------------------------------------------
def fsq_round(h: torch.Tensor, levels: torch.Tensor) -> torch.Tensor:
    """Finite scalar quantisation of one residual stage: a soft clamp to (-1 - 1/(L-1), 1 + 1/(L-1)), a hard clamp to
    [-1, 1], then rounding to the nearest of the L evenly spaced values of each lane."""
    lm1 = levels - 1.0
    soft = 1.0 + 1.0 / lm1
    c = (torch.tanh(h / soft) * soft).clamp(-1.0, 1.0)
    return torch.floor((c + 1.0) * 0.5 * lm1 + 0.5) * (2.0 / lm1) - 1.0


class CoverModules:
    def __init__(self, root: Path, device="cpu"):
        from ..io.safetensors_io import load_file

        root, self.device = Path(root), torch.device(device)
        self.dtype = _dtype_for(self.device)
        parts = {}
        for name in ("audio_tokenizer", "audio_token_detokenizer"):
            cj, wf = root / name / "config.json", root / name / VAE_FILE
            if not cj.is_file() or not wf.is_file():
                raise LoadError(f"acestep cover: {root} lacks {name}/config.json or {name}/{VAE_FILE}")
            cfg = EncoderConfig.from_json(json.loads(cj.read_text(encoding="utf-8")))
            if int(cfg.extra.get("pool_window_size", 0)) <= 0:
                raise LoadError(f"acestep cover: {name} pool_window_size must be > 0")
            parts[name] = (cfg, nd.WeightBag(load_file(wf), self.dtype, self.device))
        (self.tok_cfg, self.tok), (self.det_cfg, self.det) = parts["audio_tokenizer"], parts["audio_token_detokenizer"]
        self.window = int(self.tok_cfg.extra["pool_window_size"])
        self.acoustic = int(self.tok_cfg.extra["audio_acoustic_hidden_dim"])
        self.levels = torch.tensor(self.tok_cfg.extra.get("fsq_input_levels") or FSQ_LEVELS, dtype=torch.float32,
                                   device=self.device)

    @torch.no_grad()
    def tokenize(self, src_lat: torch.Tensor, silence: torch.Tensor) -> torch.Tensor:
        """[1, L, acoustic] -> quantised tokens [1, ceil(L / window), hidden]; the tail window is filled from `silence`."""
        w, cfg, W = self.tok, self.tok_cfg, self.window
        L, C = src_lat.shape[1:]
        if C != self.acoustic:
            raise InferenceError(f"acestep audio tokenizer: source acoustic dim {C} != {self.acoustic}")
        pad = (W - L % W) % W
        if pad:
            fill = silence[:, :pad] if silence.shape[1] >= pad else src_lat.new_zeros(1, pad, C)
            src_lat = torch.cat([src_lat, fill.to(src_lat.dtype)], dim=1)
        n = src_lat.shape[1] // W
        x = w.lin(src_lat.reshape(n, W, C).to(self.dtype), "audio_acoustic_proj")
        x = w.lin(x, "attention_pooler.embed_tokens")
        x = torch.cat([w["attention_pooler.special_token"].expand(n, 1, -1), x], dim=1)
        layers = int(cfg.extra.get("num_attention_pooler_hidden_layers", 2))
        pooled = _stack(w, "attention_pooler.", cfg, x, layers)[:, 0]                    # the query token of each window
        q = fsq_round(w.lin(pooled, "quantizer.project_in").float(), self.levels)
        return w.lin(q.to(self.dtype), "quantizer.project_out").reshape(1, n, cfg.hidden_size)

    @torch.no_grad()
    def detokenize(self, tokens: torch.Tensor) -> torch.Tensor:
        """[1, N, hidden] -> [1, N * window, acoustic]."""
        w, cfg, W = self.det, self.det_cfg, self.window
        n = tokens.shape[1]
        x = w.lin(tokens.to(self.dtype), "embed_tokens").reshape(n, 1, cfg.hidden_size) + w["special_tokens"].reshape(1, W, -1)
        layers = int(cfg.extra.get("num_attention_pooler_hidden_layers", 2))
        x = w.lin(_stack(w, "", cfg, x, layers), "proj_out")
        return x.float().reshape(1, n * W, self.acoustic)


# ---- audio post-processing --------------------------------------------------------------------------------------------------
def peak_normalize(x: torch.Tensor) -> torch.Tensor:
    """Scale so the peak sits at -1 dBFS (after first bringing any overshoot back to 1)."""
    if x.numel() == 0:
        return x
    peak = x.abs().max().item()
    if peak > 1.0:
        x = x / peak
    peak = max(x.abs().max().item(), 1e-6)
    return x * (10.0 ** (-1.0 / 20.0) / peak)


def crossfade_frames(f0: int, f1: int) -> int:
    return min(MAX_CROSSFADE, max(f1 - f0, 0) // 4)


def window_alpha(f0: int, f1: int, out_frames: int, xfade: int) -> torch.Tensor:
    """Blend weight of the generated audio for frames f0..f1: 1 inside, a raised-cosine ramp of `xfade` frames at each
    edge that borders kept source audio (the ramps lie inside the window, so frames outside stay untouched)."""
    a = torch.ones(f1 - f0)
    if xfade == 0:
        return a
    ramp = 0.5 - 0.5 * torch.cos(math.pi * (torch.arange(xfade, dtype=torch.float32) + 0.5) / xfade)
    if f0 > 0:
        a[:xfade] = torch.minimum(a[:xfade], ramp)
    if f1 < out_frames:
        a[-xfade:] = torch.minimum(a[-xfade:], ramp.flip(0))
    return a


def to_channels(x: torch.Tensor, channels: int) -> torch.Tensor:
    """[frames, c] -> [frames, channels], repeating the last source channel when the source has fewer."""
    idx = [min(c, x.shape[1] - 1) for c in range(channels)]
    return x[:, idx]


def stitch(source: torch.Tensor, generated: torch.Tensor, out_frames: int, f0: int, f1: int, xfade: int) -> torch.Tensor:
    """source [S, cs], generated [G, cg] -> [out_frames, cg]: the source outside f0..f1 (zeros past its end), the
    generated audio inside, crossfaded over `xfade` frames at the inner edges."""
    ch = generated.shape[1]
    src = torch.zeros(out_frames, ch)
    n = min(source.shape[0], out_frames)
    src[:n] = to_channels(source[:n], ch)
    gen = torch.zeros(out_frames, ch)
    g = min(generated.shape[0], out_frames)
    gen[:g] = generated[:g]
    f1 = min(f1, out_frames)
    if f1 <= f0:
        return src
    alpha = torch.zeros(out_frames)
    alpha[f0:f1] = window_alpha(f0, f1, out_frames, xfade)
    return alpha[:, None] * gen + (1.0 - alpha[:, None]) * src


# ---- pipeline ---------------------------------------------------------------------------------------------------------------
@dataclass
class SynthesisParams:
    seconds: float = DEFAULT_SECONDS
    steps: int = DEFAULT_STEPS
    shift: float = DEFAULT_SHIFT
    lyrics: str = ""
    metadata: Metadata = field(default_factory=Metadata)
    seed: int = 0


def _shards(d: Path, stem: str) -> list[Path]:
    idx = d / f"{stem}.safetensors.index.json"
    if idx.is_file():
        names = sorted(set(json.loads(idx.read_text(encoding="utf-8")).get("weight_map", {}).values()))
        if not names:
            raise LoadError(f"{idx}: index lists no shards")
        return [d / n for n in names]
    if (d / f"{stem}.safetensors").is_file():
        return [d / f"{stem}.safetensors"]
    raise LoadError(f"{d}: neither {stem}.safetensors.index.json nor {stem}.safetensors present")


def _load_shards(files: list[Path]) -> dict[str, torch.Tensor]:
    from ..io.safetensors_io import load_file

    out = {}
    for f in files:
        out.update(load_file(f))
    return out


class AceStepPipeline:
    def __init__(self, root: Path, device="cpu"):
        from ..contracts.gen_core.tokenizer import TextTokenizer, TokenizerConfig
        from ..io.safetensors_io import load_file
        from ..models.config import ModelConfig
        from ..models.text_encoders import CausalLmTextEncoder

        root = Path(root)
        self.device = torch.device(device)

        def read(rel, required=True):
            f = root / rel
            if not f.is_file():
                if not required:
                    return None
                raise LoadError(f"acestep snapshot {root} has no {rel}")
            return json.loads(f.read_text(encoding="utf-8"))

        idx = read("model_index.json")
        if idx.get("_class_name") != "AceStepPipeline":
            raise LoadError(f"{root} is not an ACE-Step snapshot (_class_name {idx.get('_class_name')!r})")
        self.vae_cfg = _from_json(VaeConfig, read("vae/config.json"), "VAE")
        self.vae_cfg.validate()
        self.dit_cfg = _from_json(TransformerConfig, read("transformer/config.json"), "transformer")
        self.dit_cfg.validate(self.vae_cfg)
        tj = read("text_encoder/config.json")
        if tj.get("use_sliding_window"):
            raise LoadError("acestep text encoder: sliding-window attention is not implemented (the pinned config has it off)")
        self.cond_cfg = EncoderConfig.from_json(read("condition_encoder/config.json"))
        if self.cond_cfg.hidden_size != self.dit_cfg.encoder_hidden_size:
            raise LoadError(f"acestep: condition encoder hidden_size {self.cond_cfg.hidden_size} != DiT "
                            f"encoder_hidden_size {self.dit_cfg.encoder_hidden_size}")
        if self.cond_cfg.extra.get("text_hidden_dim") != tj["hidden_size"]:
            raise LoadError(f"acestep: condition encoder text_hidden_dim {self.cond_cfg.extra.get('text_hidden_dim')} != "
                            f"text encoder hidden_size {tj['hidden_size']}")
        sj = read("scheduler/scheduler_config.json", required=False) or {}
        self.default_shift = float(sj.get("shift", DEFAULT_SHIFT))
        tk = root / "tokenizer" / "tokenizer.json"
        if not tk.is_file():
            raise LoadError(f"acestep snapshot {root} has no tokenizer/tokenizer.json")
        self.tokenizer = TextTokenizer.from_file(tk, TokenizerConfig(max_length=MAX_LYRIC_LEN))
        tw = _load_shards(_shards(root / "text_encoder", "model"))
        tw = {(k if k.startswith(("model.", "lm_head.")) else "model." + k): v for k, v in tw.items()}
        tcfg = ModelConfig.from_json({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", **tj})
        self.text_hidden = int(tj["hidden_size"])
        self.embed_table = tw["model.embed_tokens.weight"].float().to(self.device)
        self.text = CausalLmTextEncoder(tcfg, tw, self.device, skip_last=0, final_norm=True)
        cf = root / "condition_encoder" / VAE_FILE
        if not cf.is_file():
            cf = root / "condition_encoder" / "model.safetensors"
        if not cf.is_file():
            raise LoadError(f"acestep snapshot {root} has no condition_encoder weights")
        self.condition = ConditionEncoder(self.cond_cfg, load_file(cf), self.device)
        self.dit = AceStepDiT(self.dit_cfg, _load_shards(_shards(root / "transformer", "diffusion_pytorch_model")), self.device)
        vf = root / "vae" / VAE_FILE
        if not vf.is_file():
            raise LoadError(f"acestep snapshot {root} has no vae/{VAE_FILE}")
        self.vae = Oobleck(self.vae_cfg, load_file(vf), self.device)
        self.hop = self.vae_cfg.hop_length
        self._cover: CoverModules | None = None
        self._cover_dit: AceStepDiT | None = None

    # -- conditioning --
    def _ids(self, text: str, cap: int) -> list[int]:
        return self.tokenizer.encode_ids(text, True)[:cap] if text.strip() else []

    def latent_length(self, seconds: float) -> int:
        return int(math.ceil(seconds * self.vae_cfg.latents_per_second))

    def encode_context(self, prompt: str, lyrics: str, meta: Metadata) -> torch.Tensor:
        ids = self._ids(build_prompt(prompt, meta), MAX_TEXT_LEN)
        hidden = self.text.encode(ids).float() if ids else torch.zeros(1, 1, self.text_hidden, device=self.device)
        lyric_ids = self._ids(lyrics, MAX_LYRIC_LEN)
        lyric = self.embed_table[torch.tensor(lyric_ids, device=self.device)][None] if lyric_ids else None
        return self.condition.encode(hidden, lyric)

    # -- sampling --
    def _denoise(self, dit: AceStepDiT, context_latents, ctx, length: int, p: SynthesisParams, on_step, cancel) -> torch.Tensor:
        from ..media.seed import seeded_normal

        A = self.dit_cfg.audio_acoustic_hidden_dim
        sig = flow_sigmas(p.steps, p.shift if p.shift > 0 else self.default_shift)
        x = seeded_normal(p.seed, length * A).view(1, length, A).to(self.device)
        for k in range(len(sig) - 1):
            v = None if cancel() else dit.forward(x, context_latents, sig[k], ctx, cancel)
            if v is None:
                raise Canceled(f"{MODEL_ID}: cancelled at step {k}")
            x = x + v * (sig[k + 1] - sig[k])
            on_step(k + 1)
        return x

    def _decode(self, latents: torch.Tensor, cancel) -> torch.Tensor:
        """[1, T, acoustic] -> [frames, channels] on the host."""
        audio = self.vae.decode(latents.transpose(1, 2).contiguous(), cancel)
        if audio is None:
            raise Canceled(f"{MODEL_ID}: cancelled while decoding")
        return audio[0].t().float().cpu().contiguous()

    def _source_latents(self, source: torch.Tensor, cancel) -> torch.Tensor:
        """source [frames, c] -> [1, ceil(frames / hop), acoustic]."""
        frames = source.shape[0]
        padded = max(-(-frames // self.hop), 1) * self.hop
        planar = torch.zeros(1, self.vae_cfg.audio_channels, padded)
        planar[0, :, :frames] = to_channels(source, self.vae_cfg.audio_channels).t()
        lat = self.vae.encode(planar.to(self.device), cancel)
        if lat is None:
            raise Canceled(f"{MODEL_ID}: cancelled while encoding the source clip")
        return lat

    @torch.no_grad()
    def synthesize(self, prompt: str, p: SynthesisParams, on_step=lambda k: None, on_decode=lambda: None,
                   cancel=lambda: False) -> torch.Tensor:
        """-> [frames, 2] peak-normalised."""
        seconds = max(p.seconds, 0.1)
        T = max(self.latent_length(seconds), 1)
        A = self.dit_cfg.audio_acoustic_hidden_dim
        ctx = self.dit.embed_context(self.encode_context(prompt, p.lyrics, p.metadata))
        context_latents = torch.cat([self.condition.src_latents(T), torch.ones(1, T, A, device=self.device)], dim=-1)
        lat = self._denoise(self.dit, context_latents, ctx, T, p, on_step, cancel)
        on_decode()
        audio = self._decode(lat, cancel)
        return peak_normalize(audio[: min(int(round(self.vae_cfg.sampling_rate * seconds)), audio.shape[0])])

    def edit_window(self, task: str, start: float, end: float | None, src_frames: int, l_src: int) -> tuple[int, int, int]:
        """(target latent length, window start, window end) in latent frames."""
        lps = self.vae_cfg.latents_per_second
        src_secs = src_frames / self.vae_cfg.sampling_rate
        if task == "extend":
            if end is None:
                raise InferenceError("acestep extend: region end (the new total length in seconds) is required")
            if end <= src_secs:
                raise InferenceError(f"acestep extend: new length {end:.3f}s must exceed the source length {src_secs:.3f}s")
            target = int(math.ceil(end * lps))
            w0 = min(int(math.floor(max(start, 0.0) * lps)), l_src, target - 1)
            return target, w0, target
        target = max(l_src, 1)
        w0 = min(int(math.floor(max(start, 0.0) * lps)), target - 1)
        w1 = target if end is None else int(math.floor(end * lps))
        return target, w0, min(max(w1, w0 + 1), target)

    @torch.no_grad()
    def edit(self, prompt: str, source: torch.Tensor, task: str, start: float, end: float | None, p: SynthesisParams,
             on_step=lambda k: None, on_decode=lambda: None, cancel=lambda: False) -> torch.Tensor:
        """Regenerate latent frames w0..w1 of `source` [frames, c] (inpaint / repaint) or grow it to `end` seconds
        (extend); everything outside the window is the source, sample for sample."""
        if source.shape[0] == 0:
            raise InferenceError("acestep edit: empty source audio")
        A = self.dit_cfg.audio_acoustic_hidden_dim
        src_lat = self._source_latents(source, cancel)
        l_src = src_lat.shape[1]
        target, w0, w1 = self.edit_window(task, start, end, source.shape[0], l_src)
        silence = self.condition.src_latents(target)
        base = src_lat[:, :target] if l_src >= target else torch.cat([src_lat, silence[:, l_src:target]], dim=1)
        src_full = torch.cat([base[:, :w0], silence[:, w0:w1], base[:, w1:]], dim=1)
        mask = torch.zeros(1, target, A, device=self.device)
        mask[:, w0:w1] = 1.0
        ctx = self.dit.embed_context(self.encode_context(prompt, p.lyrics, p.metadata))
        lat = self._denoise(self.dit, torch.cat([src_full, mask], dim=-1), ctx, target, p, on_step, cancel)
        on_decode()
        gen = peak_normalize(self._decode(lat, cancel))
        out_frames = min(target * self.hop, gen.shape[0]) if task == "extend" else min(source.shape[0], gen.shape[0])
        f0, f1 = w0 * self.hop, min(w1 * self.hop, out_frames)
        return stitch(source.float(), gen, out_frames, f0, f1, crossfade_frames(f0, f1))

    def cover_modules(self, sft_root: Path) -> tuple[CoverModules, AceStepDiT]:
        if self._cover is None:
            self._cover = CoverModules(sft_root, self.device)
        if self._cover_dit is None:
            files = _shards(Path(sft_root) / "transformer", "diffusion_pytorch_model")
            self._cover_dit = AceStepDiT(self.dit_cfg, _load_shards(files), self.device)
        return self._cover, self._cover_dit

    @torch.no_grad()
    def cover(self, prompt: str, source: torch.Tensor, p: SynthesisParams, sft_root: Path, on_step=lambda k: None,
              on_decode=lambda: None, cancel=lambda: False) -> torch.Tensor:
        """Re-render `source` in the prompted style: its latents pass through the tokenizer's quantisation bottleneck,
        the de-tokenised latents become the source conditioning of the fine-tuned DiT over the whole length."""
        if source.shape[0] == 0:
            raise InferenceError("acestep cover: empty source audio")
        mods, dit = self.cover_modules(sft_root)
        A = self.dit_cfg.audio_acoustic_hidden_dim
        src_lat = self._source_latents(source, cancel)
        L = src_lat.shape[1]
        detok = mods.detokenize(mods.tokenize(src_lat, self.condition.src_latents(max(mods.window, 1))))
        src = detok[:, :L] if detok.shape[1] >= L else torch.cat([detok, self.condition.src_latents(L - detok.shape[1])], dim=1)
        ctx = dit.embed_context(self.encode_context(prompt, p.lyrics, p.metadata))
        steps = SynthesisParams(p.seconds, COVER_STEPS, p.shift, p.lyrics, p.metadata, p.seed)
        lat = self._denoise(dit, torch.cat([src, torch.ones(1, L, A, device=self.device)], dim=-1), ctx, L, steps, on_step, cancel)
        on_decode()
        gen = peak_normalize(self._decode(lat, cancel))
        return gen[: min(source.shape[0], gen.shape[0])]


# ---- generator --------------------------------------------------------------------------------------------------------------
def acestep_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family=FAMILY, backend=backend, modality=Modality.AUDIO,
        capabilities=Capabilities(
            supports_negative_prompt=False, supports_guidance=False, supports_true_cfg=False,
            conditioning=[ConditioningKind.AUDIO_EDIT], supports_lora=False, supports_lokr=False, samplers=[], schedulers=[],
            supported_guidance_methods=[], min_size=0, max_size=0, max_count=1, audio_sample_rates=[SAMPLE_RATE],
            max_audio_duration_secs=MAX_DURATION_SECS, audio_voices=[], audio_languages=list(LANGUAGES),
            audio_edit_modes=list(EDIT_MODES)),
        required_components=[])


def _audio_edit(req: GenerationRequest):
    return next((c for c in req.conditioning if c.kind is ConditioningKind.AUDIO_EDIT), None)


class AceStepGenerator(Generator):
    def __init__(self, root: Path, backend: str, prefix: str = "", sft_cover_root: Path | None = None):
        self.root, self.backend, self.sft_cover_root = Path(root), backend, sft_cover_root
        self._descriptor = acestep_descriptor(backend, prefix)
        self._pipe: AceStepPipeline | None = None

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        if not req.prompt.strip():
            raise InferenceError(f"{mid}: prompt (the music style description) must not be empty")
        if req.steps is not None and req.steps > MAX_STEPS:
            raise InferenceError(f"{mid}: steps {req.steps} above the {MAX_STEPS}-step ceiling")
        if req.scheduler_shift is not None and not (math.isfinite(req.scheduler_shift) and req.scheduler_shift > 0):
            raise InferenceError(f"{mid}: scheduler_shift (flow-match sigma shift) must be > 0, got {req.scheduler_shift}")
        a = req.audio
        if a is not None:
            if a.bpm is not None and not (math.isfinite(a.bpm) and a.bpm > 0):
                raise InferenceError(f"{mid}: audio.bpm must be finite and > 0, got {a.bpm}")
            if a.target_duration is not None and a.target_duration < 0.04:
                raise InferenceError(f"{mid}: audio.target_duration {a.target_duration}s below the 0.04 s floor (25 fps latents)")
        edit = _audio_edit(req)
        if edit is not None:
            src = edit.audio
            if src is None or src.channels == 0 or not src.samples:
                raise InferenceError(f"{mid}: audio edit source clip is empty")
            if src.sample_rate != SAMPLE_RATE:
                raise Unsupported(f"{mid}: audio edit source must be {SAMPLE_RATE} Hz (the model's native rate), got {src.sample_rate}")
            secs = (len(src.samples) // src.channels) / src.sample_rate
            start, end = edit.region if edit.region is not None else (None, None)
            if edit.mode == "extend":
                if end is None:
                    raise InferenceError(f"{mid}: extend requires region end_secs (the new total length in seconds)")
                if end <= secs:
                    raise InferenceError(f"{mid}: extend length {end}s must exceed the source length {secs:.3f}s")
            elif edit.mode in ("inpaint", "repaint"):
                if edit.region is None:
                    raise InferenceError(f"{mid}: {edit.mode} editing requires a region (start/end seconds)")
                if start >= secs:
                    raise InferenceError(f"{mid}: audio edit region start {start}s is at/beyond the {secs:.3f}s clip")
                if end is not None and end > secs + 1e-3:
                    raise InferenceError(f"{mid}: audio edit region end {end}s is beyond the {secs:.3f}s clip")
        self._descriptor.capabilities.validate_request_audio(mid, req)

    def pipeline(self) -> AceStepPipeline:
        if self._pipe is None:
            self._pipe = AceStepPipeline(self.root, "cuda" if self.backend == "b200" else "cpu")
        return self._pipe

    def _cover_root(self) -> Path:
        if self.sft_cover_root is None:
            raise InferenceError(
                f"{self._descriptor.id} cover needs the fine-tuned checkpoint staged as the '{COVER_COMPONENT}' component: a "
                "snapshot directory with audio_tokenizer/, audio_token_detokenizer/ and transformer/ passed in the load "
                "spec's components; it is never fetched implicitly")
        return self.sft_cover_root

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        self.validate(req)
        if req.cancel.is_cancelled():
            raise Canceled(f"{self._descriptor.id}: cancelled")
        from ..media.seed import default_seed

        edit = _audio_edit(req)
        if edit is not None and edit.mode == "cover":
            self._cover_root()
        a = req.audio
        p = SynthesisParams(
            seconds=a.target_duration if a is not None and a.target_duration is not None else DEFAULT_SECONDS,
            steps=req.steps if req.steps is not None else DEFAULT_STEPS,
            shift=req.scheduler_shift if req.scheduler_shift is not None else DEFAULT_SHIFT,
            lyrics=(a.lyrics or "") if a is not None else "",
            metadata=Metadata(a.bpm, a.musical_key, None, a.language) if a is not None else Metadata(),
            seed=req.seed if req.seed is not None else default_seed())
        pipe = self.pipeline()
        total = COVER_STEPS if edit is not None and edit.mode == "cover" else p.steps
        hooks = dict(on_step=lambda k: on_progress(ProgressStep(k, total)), on_decode=lambda: on_progress(ProgressDecoding()),
                     cancel=req.cancel.is_cancelled)
        if edit is None:
            out = pipe.synthesize(req.prompt, p, **hooks)
        else:
            src = torch.tensor(edit.audio.samples, dtype=torch.float32).view(-1, edit.audio.channels)
            if edit.mode == "cover":
                out = pipe.cover(req.prompt, src, p, self._cover_root(), **hooks)
            else:
                start, end = edit.region if edit.region is not None else (0.0, None)
                out = pipe.edit(req.prompt, src, edit.mode, start, end, p, **hooks)
        return GenerationOutput(audio=AudioTrack(SAMPLE_RATE, CHANNELS, out.reshape(-1).tolist()))


def registration(backend: str) -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> AceStepGenerator:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise LoadError(f"{mid} expects a diffusers snapshot directory (model_index.json + transformer/ + "
                            "condition_encoder/ + text_encoder/ + tokenizer/ + vae/), not a single file")
        if spec.quantize is not None:
            raise Unsupported(f"{mid} does not support on-the-fly quantization")
        if spec.adapters:
            raise Unsupported(f"{mid} does not support LoRA/LoKr adapters")
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid} does not support control/IP-adapter overlays")
        unknown = sorted(set(spec.components) - {COVER_COMPONENT})
        if unknown:
            raise LoadError(f"{mid}: unknown components {unknown} (accepted: ['{COVER_COMPONENT}'])")
        sft = spec.components.get(COVER_COMPONENT)
        if sft is not None and sft.is_file:
            raise LoadError(f"{mid} component '{COVER_COMPONENT}' must be the fine-tuned snapshot directory (audio_tokenizer/ + "
                            f"audio_token_detokenizer/ + transformer/), not the file {sft.path}")
        return AceStepGenerator(Path(spec.weights.path), backend, prefix, Path(sft.path) if sft is not None else None)

    return Registration(descriptor=lambda: acestep_descriptor(backend, prefix), load=load)


# ---- synthetic snapshot -----------------------------------------------------------------------------------------------------
def _layer_weights(w: dict, p: str, cfg: EncoderConfig, rn, lin) -> None:
    H, KV, D, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size
    for n, o, i in (("to_q", H * D, d), ("to_k", KV * D, d), ("to_v", KV * D, d), ("to_out.0", d, H * D)):
        lin(w, p + "self_attn." + n, o, i, bias=False)
    for n in ("norm_q", "norm_k"):
        w[p + f"self_attn.{n}.weight"] = 1.0 + 0.1 * rn(D)
    for n in ("input_layernorm", "post_attention_layernorm"):
        w[p + n + ".weight"] = 1.0 + 0.1 * rn(d)
    lin(w, p + "mlp.gate_proj", cfg.intermediate_size, d, bias=False)
    lin(w, p + "mlp.up_proj", cfg.intermediate_size, d, bias=False)
    lin(w, p + "mlp.down_proj", d, cfg.intermediate_size, bias=False)


def random_condition_weights(cfg: EncoderConfig, silence_len: int = 12, seed: int = 0) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    e = cfg.extra
    lin(w, "text_projector", cfg.hidden_size, e["text_hidden_dim"], bias=False)
    for name, in_dim, layers in (("lyric_encoder.", e["text_hidden_dim"], e["num_lyric_encoder_hidden_layers"]),
                                 ("timbre_encoder.", e["timbre_hidden_dim"], e["num_timbre_encoder_hidden_layers"])):
        lin(w, name + "embed_tokens", cfg.hidden_size, in_dim)
        for i in range(layers):
            _layer_weights(w, f"{name}layers.{i}.", cfg, rn, lin)
        w[name + "norm.weight"] = 1.0 + 0.1 * rn(cfg.hidden_size)
    w["timbre_encoder.special_token"] = rn(1, 1, cfg.hidden_size) * 0.5
    w["silence_latent"] = rn(1, silence_len, e["timbre_hidden_dim"]) * 0.3
    return w


def random_dit_weights(cfg: TransformerConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    d, H, KV, D = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    w["proj_in_conv.weight"] = rn(d, cfg.in_channels, cfg.patch_size) * 0.05
    w["proj_in_conv.bias"] = rn(d) * 0.05
    w["proj_out_conv.weight"] = rn(d, cfg.audio_acoustic_hidden_dim, cfg.patch_size) * 0.05
    w["proj_out_conv.bias"] = rn(cfg.audio_acoustic_hidden_dim) * 0.05
    for te in ("time_embed.", "time_embed_r."):
        lin(w, te + "linear_1", d, FREQ_DIM)
        lin(w, te + "linear_2", d, d)
        lin(w, te + "time_proj", 6 * d, d)
    lin(w, "condition_embedder", d, cfg.encoder_hidden_size)
    for i in range(cfg.num_hidden_layers):
        b = f"layers.{i}."
        for a in ("self_attn.", "cross_attn."):
            for n, o, ic in (("to_q", H * D, d), ("to_k", KV * D, d), ("to_v", KV * D, d), ("to_out.0", d, H * D)):
                lin(w, b + a + n, o, ic, bias=cfg.attention_bias)
            w[b + a + "norm_q.weight"] = 1.0 + 0.1 * rn(D)
            w[b + a + "norm_k.weight"] = 1.0 + 0.1 * rn(D)
        for n in ("self_attn_norm", "cross_attn_norm", "mlp_norm"):
            w[b + n + ".weight"] = 1.0 + 0.1 * rn(d)
        lin(w, b + "mlp.gate_proj", cfg.intermediate_size, d, bias=False)
        lin(w, b + "mlp.up_proj", cfg.intermediate_size, d, bias=False)
        lin(w, b + "mlp.down_proj", d, cfg.intermediate_size, bias=False)
        w[b + "scale_shift_table"] = rn(1, 6, d) * 0.1
    w["norm_out.weight"] = 1.0 + 0.1 * rn(d)
    w["scale_shift_table"] = rn(1, 2, d) * 0.1
    return w


def random_oobleck_weights(cfg: VaeConfig, encoder_hidden: int = 8, seed: int = 0) -> dict[str, torch.Tensor]:
    """Weight-normed tensors (magnitude + direction) for both halves, channel widths following the config's multiples."""
    rn, _ = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}

    def conv(p, o, i, k, transposed=False):
        v = rn(i, o, k) if transposed else rn(o, i, k)
        w[p + ".weight_v"] = v
        w[p + ".weight_g"] = (1.0 + 0.1 * rn(v.shape[0], 1, 1)) * (0.8 * math.sqrt(v[0].numel() / (i * k)))
        w[p + ".bias"] = rn(o) * 0.02

    def snk(p, c):
        w[p + ".alpha"] = rn(1, c, 1) * 0.1
        w[p + ".beta"] = rn(1, c, 1) * 0.1

    def res(p, c):
        snk(p + ".snake1", c)
        conv(p + ".conv1", c, c, 7)
        snk(p + ".snake2", c)
        conv(p + ".conv2", c, c, 1)

    mult, ratios, latent = cfg.channel_multiples, cfg.downsampling_ratios, cfg.decoder_input_channels
    dc = cfg.decoder_channels
    widths = [dc * m for m in reversed(mult)] + [dc]                  # decoder: widest first
    conv("decoder.conv1", widths[0], latent, 7)
    for i, s in enumerate(reversed(ratios)):
        b = f"decoder.block.{i}"
        snk(b + ".snake1", widths[i])
        conv(b + ".conv_t1", widths[i + 1], widths[i], 2 * s, transposed=True)
        for j in range(3):
            res(f"{b}.res_unit{j + 1}", widths[i + 1])
    snk("decoder.snake1", dc)
    conv("decoder.conv2", cfg.audio_channels, dc, 7)
    w.pop("decoder.conv2.bias")
    ew = [encoder_hidden] + [encoder_hidden * m for m in mult]
    conv("encoder.conv1", ew[0], cfg.audio_channels, 7)
    for i, s in enumerate(ratios):
        b = f"encoder.block.{i}"
        for j in range(3):
            res(f"{b}.res_unit{j + 1}", ew[i])
        snk(b + ".snake1", ew[i])
        conv(b + ".conv1", ew[i + 1], ew[i], 2 * s)
    snk("encoder.snake1", ew[-1])
    conv("encoder.conv2", 2 * latent, ew[-1], 3)
    return w


SYNTH_VAE = {"_class_name": "AutoencoderOobleck", "audio_channels": 2, "channel_multiples": [1, 2], "decoder_channels": 8,
             "decoder_input_channels": 8, "downsampling_ratios": [2, 4], "encoder_hidden_size": 8, "sampling_rate": 48000}
SYNTH_DIT = {"in_channels": 24, "audio_acoustic_hidden_dim": 8, "encoder_hidden_size": 32, "hidden_size": 64,
             "intermediate_size": 96, "head_dim": 16, "num_attention_heads": 4, "num_key_value_heads": 2,
             "num_hidden_layers": 2, "patch_size": 2, "layer_types": ["sliding_attention", "full_attention"],
             "sliding_window": 4, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "is_turbo": True}
SYNTH_COND = {"hidden_size": 32, "intermediate_size": 48, "head_dim": 8, "num_attention_heads": 4, "num_key_value_heads": 2,
              "num_lyric_encoder_hidden_layers": 1, "num_timbre_encoder_hidden_layers": 1, "text_hidden_dim": 32,
              "timbre_hidden_dim": 8, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "sliding_window": 4}
SYNTH_TOK = {"hidden_size": 32, "intermediate_size": 48, "head_dim": 8, "num_attention_heads": 4, "num_key_value_heads": 2,
             "num_attention_pooler_hidden_layers": 1, "pool_window_size": 5, "audio_acoustic_hidden_dim": 8,
             "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "fsq_input_levels": [8, 8, 8, 5, 5, 5], "fsq_dim": 32}


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny complete snapshot (hop 8 instead of 1920, so a second of audio is 6000 latent frames: keep requests short)."""
    from ..io.safetensors_io import save_file
    from ..media.z_image import _write_synthetic_qwen3

    root = Path(root)
    for sub in ("vae", "transformer", "condition_encoder", "scheduler"):
        (root / sub).mkdir(parents=True, exist_ok=True)
    (root / "model_index.json").write_text(json.dumps({"_class_name": "AceStepPipeline"}))
    for sub, cfg in (("vae", SYNTH_VAE), ("transformer", SYNTH_DIT), ("condition_encoder", SYNTH_COND)):
        (root / sub / "config.json").write_text(json.dumps(cfg))
    (root / "scheduler" / "scheduler_config.json").write_text(json.dumps({"_class_name": "FlowMatchEulerDiscreteScheduler", "shift": 3.0}))
    _write_synthetic_qwen3(root, SYNTH_COND["text_hidden_dim"], 8, seed + 1)
    save_file(random_condition_weights(EncoderConfig.from_json(SYNTH_COND), seed=seed + 2), root / "condition_encoder" / VAE_FILE)
    save_file(random_dit_weights(_from_json(TransformerConfig, SYNTH_DIT, "transformer"), seed + 3),
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    save_file(random_oobleck_weights(_from_json(VaeConfig, SYNTH_VAE, "VAE"), seed=seed + 4), root / "vae" / VAE_FILE)
    return root


def write_synthetic_cover_snapshot(root, seed: int = 0) -> Path:
    from ..io.safetensors_io import save_file

    root = Path(root)
    cfg = EncoderConfig.from_json(SYNTH_TOK)
    rn, lin = nd.randn_weights(seed + 10)
    h, A, W = cfg.hidden_size, SYNTH_TOK["audio_acoustic_hidden_dim"], SYNTH_TOK["pool_window_size"]
    tok: dict[str, torch.Tensor] = {}
    lin(tok, "audio_acoustic_proj", h, A)
    lin(tok, "attention_pooler.embed_tokens", h, h)
    tok["attention_pooler.special_token"] = rn(1, 1, h) * 0.5
    _layer_weights(tok, "attention_pooler.layers.0.", cfg, rn, lin)
    tok["attention_pooler.norm.weight"] = 1.0 + 0.1 * rn(h)
    lin(tok, "quantizer.project_in", len(FSQ_LEVELS), h, std=0.3)
    lin(tok, "quantizer.project_out", h, len(FSQ_LEVELS), std=0.3)
    det: dict[str, torch.Tensor] = {}
    lin(det, "embed_tokens", h, h)
    det["special_tokens"] = rn(1, W, h) * 0.5
    _layer_weights(det, "layers.0.", cfg, rn, lin)
    det["norm.weight"] = 1.0 + 0.1 * rn(h)
    lin(det, "proj_out", A, h)
    for name, w in (("audio_tokenizer", tok), ("audio_token_detokenizer", det)):
        (root / name).mkdir(parents=True, exist_ok=True)
        (root / name / "config.json").write_text(json.dumps(SYNTH_TOK))
        save_file(w, root / name / VAE_FILE)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    save_file(random_dit_weights(_from_json(TransformerConfig, SYNTH_DIT, "transformer"), seed + 11),
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    return root
