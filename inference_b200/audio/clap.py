"""CLAP (`laion/clap-htsat-unfused`): a joint audio-text embedding space (the reference's candle-audio-clap crate:
src/mel.rs, src/audio.rs, src/text.rs, src/model.rs).

Audio side: 48 kHz mono, repeat-padded / truncated to 10 s, Slaney log-mel (n_fft 1024, hop 480, 64 bands, 50 Hz -
14 kHz, power in dB) -> HTSAT, a Swin transformer over the spectrogram folded into a square image: 4x4 patch
embedding, stages of windowed self-attention with relative-position bias (every second block on windows shifted by
half a window, with the wrap-around masked), patch merging between stages, LayerNorm, mean over all tokens.
Text side: RoBERTa with its tanh pooler. Each tower ends in a two-layer projection; vectors are L2-normalised, so a
dot product between an audio and a text vector is their similarity. Weight names follow the Hugging Face `ClapModel`
checkpoint. Projections run on the tcgen05 GEMM for bf16 weights on a CUDA device."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from ..contracts.gen_core.media import AudioTrack
from ..contracts.gen_core.traits import AudioEmbedder, SimpleDescriptor
from ..models.text_encoders import linear
from .dsp import AudioError, hann_window
from .mel import slaney_filterbank
from .whisper import to_mono

SAMPLE_RATE = 48_000
N_FFT, HOP, N_MELS = 1024, 480, 64
F_MIN, F_MAX = 50.0, 14_000.0
MAX_SAMPLES = 10 * SAMPLE_RATE


# ---- front end ---------------------------------------------------------------------------------------------------------
def resample_linear(samples: torch.Tensor, src_rate: int, dst_rate: int = SAMPLE_RATE) -> torch.Tensor:
    if src_rate == dst_rate or samples.numel() == 0:
        return samples
    ratio = dst_rate / src_rate
    n = int(round(samples.numel() * ratio))
    pos = torch.arange(n, dtype=torch.float64) / ratio
    left = pos.floor().long()
    frac = (pos - left).float()
    last = samples.numel() - 1
    a, b = samples[left.clamp(max=last)], samples[(left + 1).clamp(max=last)]
    return a + (b - a) * frac


def fit_length(wav: torch.Tensor, n: int = MAX_SAMPLES) -> torch.Tensor:
    """Longer clips keep their first n samples; shorter ones are tiled a whole number of times, then zero-padded."""
    if wav.numel() >= n:
        return wav[:n]
    rep = n // wav.numel()
    return F.pad(wav.repeat(rep), (0, n - rep * wav.numel()))


def log_mel_db(wav: torch.Tensor) -> torch.Tensor:
    """[frames, 64] log-mel in dB (10 log10 of the mel power, floor 1e-10)."""
    spec = torch.stft(wav.float(), N_FFT, HOP, window=hann_window(N_FFT), center=True, pad_mode="reflect",
                      return_complex=True)
    mel = slaney_filterbank(SAMPLE_RATE, N_FFT, N_MELS, F_MIN, F_MAX) @ (spec.abs() ** 2)
    return (10.0 * torch.log10(mel.clamp(min=1e-10))).t().contiguous()


def track_features(track: AudioTrack) -> torch.Tensor:
    """[1, 1, frames, 64] input features of one clip."""
    if not track.samples:
        raise AudioError("clap: empty audio")
    wav = resample_linear(to_mono(torch.tensor(track.samples, dtype=torch.float32), track.channels), track.sample_rate)
    return log_mel_db(fit_length(wav))[None, None]


# ---- HTSAT audio tower -----------------------------------------------------------------------------------------------------
@dataclass
class ClapAudioConfig:
    spec_size: int = 256
    num_mel_bins: int = 64
    patch_size: int = 4
    patch_stride: int = 4
    patch_embeds_hidden_size: int = 96
    depths: list[int] = field(default_factory=lambda: [2, 2, 6, 2])
    num_attention_heads: list[int] = field(default_factory=lambda: [4, 8, 16, 32])
    window_size: int = 8
    mlp_ratio: float = 4.0
    layer_norm_eps: float = 1e-5
    hidden_size: int = 768
    projection_dim: int = 512
    enable_patch_layer_norm: bool = True

    @staticmethod
    def from_json(j: dict) -> "ClapAudioConfig":
        a = j.get("audio_config", j)
        keys = ClapAudioConfig.__dataclass_fields__
        c = ClapAudioConfig(**{k: a[k] for k in keys if k in a})
        if "projection_dim" in j:
            c.projection_dim = j["projection_dim"]
        return c


def _window_partition(x: torch.Tensor, ws: int) -> torch.Tensor:
    b, h, w, c = x.shape
    return x.view(b, h // ws, ws, w // ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(-1, ws * ws, c)


def _window_reverse(win: torch.Tensor, ws: int, h: int, w: int) -> torch.Tensor:
    c = win.shape[-1]
    return win.view(-1, h // ws, w // ws, ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(-1, h, w, c)


def _relative_position_index(ws: int) -> torch.Tensor:
    coords = torch.stack(torch.meshgrid(torch.arange(ws), torch.arange(ws), indexing="ij")).flatten(1)
    rel = (coords[:, :, None] - coords[:, None, :]).permute(1, 2, 0).contiguous()
    rel[:, :, 0] += ws - 1
    rel[:, :, 1] += ws - 1
    rel[:, :, 0] *= 2 * ws - 1
    return rel.sum(-1)


def _shift_mask(h: int, w: int, ws: int, shift: int, device) -> torch.Tensor:
    """Additive mask [windows, ws*ws, ws*ws]: tokens that were not neighbours before the cyclic shift do not attend."""
    img = torch.zeros(1, h, w, 1, device=device)
    cnt = 0
    for hs in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
        for wsl in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
            img[:, hs, wsl, :] = cnt
            cnt += 1
    m = _window_partition(img, ws).squeeze(-1)
    d = m.unsqueeze(1) - m.unsqueeze(2)
    return torch.where(d != 0, torch.full_like(d, -100.0), torch.zeros_like(d))


class ClapAudioTower:
    def __init__(self, cfg: ClapAudioConfig, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        pre = "audio_model.audio_encoder."
        self.w = {k[len(pre):]: v.to(self.device, dtype if v.is_floating_point() else v.dtype).contiguous()
                  for k, v in weights.items() if k.startswith(pre)}
        self.proj = {k[len("audio_projection."):]: v.to(self.device, dtype) for k, v in weights.items()
                     if k.startswith("audio_projection.")}
        self.freq_ratio = cfg.spec_size // cfg.num_mel_bins
        self._rel_index: dict[int, torch.Tensor] = {}

    def _ln(self, x, name):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(),
                            self.cfg.layer_norm_eps).to(self.dtype)

    def _mel_to_image(self, x: torch.Tensor) -> torch.Tensor:
        """[B, 1, T, F] -> [B, 1, F * ratio, T / ratio]: the time axis is cut into `ratio` strips stacked along frequency."""
        c = self.cfg
        _, _, t, f = x.shape
        width, height = c.spec_size * self.freq_ratio, c.spec_size // self.freq_ratio
        if t > width or f > height:
            raise AudioError("clap: the spectrogram is larger than the model's input")
        if t < width:
            x = F.interpolate(x, (width, f), mode="bicubic", align_corners=True)
        if f < height:
            x = F.interpolate(x, (x.shape[2], height), mode="bicubic", align_corners=True)
        b, ch, t, f = x.shape
        r = self.freq_ratio
        x = x.reshape(b, ch * r, t // r, f).permute(0, 1, 3, 2).contiguous()
        return x.reshape(b, ch, f * r, t // r)

    def _block(self, x, p, dims, heads, shift):
        c = self.cfg
        h, w = dims
        ws = c.window_size
        if min(dims) <= ws:
            ws, shift = min(dims), 0
        b, _, ch = x.shape
        y = self._ln(x, p + "layernorm_before").view(b, h, w, ch)
        pr, pb = (ws - w % ws) % ws, (ws - h % ws) % ws
        y = F.pad(y, (0, 0, 0, pr, 0, pb))
        hp, wp = h + pb, w + pr
        if shift > 0:
            y = torch.roll(y, shifts=(-shift, -shift), dims=(1, 2))
        win = _window_partition(y, ws)
        a = p + "attention.self."
        q, k, v = (linear(win, self.w[a + n + ".weight"], self.w.get(a + n + ".bias")) for n in ("query", "key", "value"))
        sp = lambda t: t.view(t.shape[0], ws * ws, heads, ch // heads).transpose(1, 2).float()
        scores = sp(q) @ sp(k).transpose(-1, -2) / math.sqrt(ch // heads)
        idx = self._rel_index.setdefault(ws, _relative_position_index(ws).to(self.device))
        bias = self.w[a + "relative_position_bias_table"].float()[idx.view(-1)].view(ws * ws, ws * ws, -1).permute(2, 0, 1)
        scores = scores + bias.unsqueeze(0)
        if shift > 0:
            m = _shift_mask(hp, wp, ws, shift, self.device)
            nw = m.shape[0]
            scores = (scores.view(-1, nw, heads, ws * ws, ws * ws) + m[None, :, None]).view(-1, heads, ws * ws, ws * ws)
        ctx = (torch.softmax(scores, -1) @ sp(v)).transpose(1, 2).reshape(-1, ws * ws, ch).to(self.dtype)
        ctx = linear(ctx, self.w[p + "attention.output.dense.weight"], self.w[p + "attention.output.dense.bias"])
        y = _window_reverse(ctx, ws, hp, wp)
        if shift > 0:
            y = torch.roll(y, shifts=(shift, shift), dims=(1, 2))
        x = x + y[:, :h, :w].reshape(b, h * w, ch)
        z = self._ln(x, p + "layernorm_after")
        z = F.gelu(linear(z, self.w[p + "intermediate.dense.weight"], self.w[p + "intermediate.dense.bias"]).float())
        return x + linear(z.to(self.dtype), self.w[p + "output.dense.weight"], self.w[p + "output.dense.bias"])

    def _merge(self, x, p, dims):
        h, w = dims
        b, _, ch = x.shape
        y = F.pad(x.view(b, h, w, ch), (0, 0, 0, w % 2, 0, h % 2))
        y = torch.cat([y[:, 0::2, 0::2], y[:, 1::2, 0::2], y[:, 0::2, 1::2], y[:, 1::2, 1::2]], -1).reshape(b, -1, 4 * ch)
        return linear(self._ln(y, p + "norm"), self.w[p + "reduction.weight"])

    @torch.no_grad()
    def pooled(self, feats: torch.Tensor) -> torch.Tensor:
        """feats [B, 1, T, F] log-mel -> [B, hidden]."""
        c = self.cfg
        x = feats.to(self.device, self.dtype)
        bn = lambda n: self.w["batch_norm." + n].float()
        x = ((x.float() - bn("running_mean")) / torch.sqrt(bn("running_var") + 1e-5) * bn("weight") + bn("bias")).to(self.dtype)
        img = self._mel_to_image(x)
        pad = (c.patch_size - c.patch_stride) // 2
        x = F.conv2d(img, self.w["patch_embed.proj.weight"], self.w["patch_embed.proj.bias"], stride=c.patch_stride,
                     padding=pad).flatten(2).transpose(1, 2)
        if c.enable_patch_layer_norm:
            x = self._ln(x, "patch_embed.norm")
        grid = c.spec_size // c.patch_stride
        dims = (grid, grid)
        for s, (depth, heads) in enumerate(zip(c.depths, c.num_attention_heads)):
            for i in range(depth):
                x = self._block(x, f"layers.{s}.blocks.{i}.", dims, heads, 0 if i % 2 == 0 else c.window_size // 2)
            if s < len(c.depths) - 1:
                x = self._merge(x, f"layers.{s}.downsample.", dims)
                dims = ((dims[0] + 1) // 2, (dims[1] + 1) // 2)
        return self._ln(x, "norm").float().mean(dim=1).to(self.dtype)

    @torch.no_grad()
    def embed(self, feats: torch.Tensor) -> torch.Tensor:
        h = self.pooled(feats)
        h = F.relu(linear(h, self.proj["linear1.weight"], self.proj["linear1.bias"]).float()).to(self.dtype)
        return F.normalize(linear(h, self.proj["linear2.weight"], self.proj["linear2.bias"]).float(), dim=-1)


# ---- RoBERTa text tower ------------------------------------------------------------------------------------------------------
@dataclass
class ClapTextConfig:
    vocab_size: int = 50265
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 514
    layer_norm_eps: float = 1e-12
    pad_token_id: int = 1

    @staticmethod
    def from_json(j: dict) -> "ClapTextConfig":
        t = j.get("text_config", j)
        keys = ClapTextConfig.__dataclass_fields__
        return ClapTextConfig(**{k: t[k] for k in keys if k in t})


class ClapTextTower:
    def __init__(self, cfg: ClapTextConfig, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k[len("text_model."):]: v.to(self.device, dtype if v.is_floating_point() else v.dtype).contiguous()
                  for k, v in weights.items() if k.startswith("text_model.")}
        self.proj = {k[len("text_projection."):]: v.to(self.device, dtype) for k, v in weights.items()
                     if k.startswith("text_projection.")}

    def _ln(self, x, name):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(),
                            self.cfg.layer_norm_eps).to(self.dtype)

    @torch.no_grad()
    def embed(self, ids: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
        """ids [B, L] (RoBERTa ids, padded with pad_token_id) -> unit vectors [B, projection_dim]."""
        c = self.cfg
        ids = ids.to(self.device)
        keep = (ids != c.pad_token_id) if mask is None else mask.to(self.device).bool()
        pos = torch.cumsum(keep.long(), dim=1) * keep.long() + c.pad_token_id      # RoBERTa: positions count real tokens
        e = "embeddings."
        x = self.w[e + "word_embeddings.weight"][ids] + self.w[e + "position_embeddings.weight"][pos] + \
            self.w[e + "token_type_embeddings.weight"][0]
        x = self._ln(x, e + "LayerNorm")
        B, L, E = x.shape
        H = c.num_attention_heads
        add = torch.zeros(B, 1, 1, L, device=self.device).masked_fill(~keep[:, None, None, :], float("-inf"))
        for i in range(c.num_hidden_layers):
            p = f"encoder.layer.{i}."
            q, k, v = (linear(x, self.w[f"{p}attention.self.{n}.weight"], self.w[f"{p}attention.self.{n}.bias"])
                       .view(B, L, H, E // H).transpose(1, 2).float() for n in ("query", "key", "value"))
            a = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(E // H) + add, -1) @ v
            a = a.transpose(1, 2).reshape(B, L, E).to(self.dtype)
            a = linear(a, self.w[p + "attention.output.dense.weight"], self.w[p + "attention.output.dense.bias"])
            x = self._ln(a + x, p + "attention.output.LayerNorm")
            h = F.gelu(linear(x, self.w[p + "intermediate.dense.weight"], self.w[p + "intermediate.dense.bias"]).float())
            h = linear(h.to(self.dtype), self.w[p + "output.dense.weight"], self.w[p + "output.dense.bias"])
            x = self._ln(h + x, p + "output.LayerNorm")
        pooled = torch.tanh(linear(x[:, 0], self.w["pooler.dense.weight"], self.w["pooler.dense.bias"]).float())
        h = F.relu(linear(pooled.to(self.dtype), self.proj["linear1.weight"], self.proj["linear1.bias"]).float())
        return F.normalize(linear(h.to(self.dtype), self.proj["linear2.weight"], self.proj["linear2.bias"]).float(), dim=-1)


# ---- provider ----------------------------------------------------------------------------------------------------------------
class ClapAudioEmbedder(AudioEmbedder):
    ID = "clap_htsat_unfused"

    def __init__(self, audio: ClapAudioTower, text: ClapTextTower | None, tokenizer, backend: str):
        self.audio, self.text, self.tok, self.backend = audio, text, tokenizer, backend

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "clap", self.backend, {"dim": self.audio.cfg.projection_dim,
                                                                "sample_rate": SAMPLE_RATE, "joint_text": self.text is not None})

    def embed(self, audio: list[AudioTrack]) -> list[list[float]]:
        if not audio:
            return []
        feats = torch.cat([track_features(t) for t in audio], dim=0)
        return self.audio.embed(feats).cpu().tolist()

    def embed_text(self, texts: list[str], max_length: int = 77) -> list[list[float]]:
        """Text queries in the same space (cosine against `embed` ranks clips by a description)."""
        if self.text is None or self.tok is None:
            raise AudioError("clap: this snapshot was loaded without its text tower")
        if not texts:
            return []
        pad = self.text.cfg.pad_token_id
        rows = [self.tok.encode(t, add_special_tokens=True)[:max_length] for t in texts]
        L = max(len(r) for r in rows)
        ids = torch.tensor([r + [pad] * (L - len(r)) for r in rows], dtype=torch.long)
        return self.text.embed(ids).cpu().tolist()
