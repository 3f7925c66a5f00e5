"""Chatterbox voice encoder: a GE2E-style speaker verifier that maps a few seconds of reference audio to a
256-dimensional speaker-identity vector (the reference's candle-audio-chatterbox-ve crate: src/frontend.rs,
src/encoder.rs, src/model.rs).

Front end: resample to 16 kHz, raise quiet clips to -30 dBFS (never attenuate), power STFT (n_fft 400, hop 160,
periodic Hann, reflect padding), 40-band Slaney mel of the raw power. Encoder: 3-layer LSTM (hidden 256), the last
hidden state through a 256 -> 256 projection + ReLU; clips longer than 160 frames are cut into half-overlapping
160-frame partials whose embeddings are averaged, then L2-normalised. Weights: `ve.safetensors`
(`lstm.weight_ih_l0`, ..., `proj.weight`, `proj.bias`)."""
from __future__ import annotations

import math

import torch

from ..contracts.errors import LoadError
from ..contracts.gen_core.media import AudioTrack
from ..contracts.gen_core.traits import SimpleDescriptor, VoiceEmbedder
from .dsp import AudioError, hann_window
from .mel import slaney_filterbank
from .whisper import resample_to_16k, to_mono

SAMPLE_RATE = 16_000
N_FFT, HOP, N_MELS = 400, 160, 40
HIDDEN, NUM_LAYERS, EMBED_DIM = 256, 3, 256
PARTIALS_N_FRAMES = 160
AUDIO_NORM_TARGET_DBFS = -30.0


def normalize_volume(wav: torch.Tensor) -> torch.Tensor:
    """Gain up to the target loudness; louder clips are left alone."""
    if wav.numel() == 0:
        return wav
    mean_sq = float((wav * wav).mean())
    if mean_sq <= 0:
        return wav
    change = AUDIO_NORM_TARGET_DBFS - 10.0 * math.log10(mean_sq)
    return wav if change <= 0 else wav * (10.0 ** (change / 20.0))


def wav_to_mel_frames(samples: torch.Tensor, src_rate: int) -> torch.Tensor:
    """[frames, 40] raw-power mel."""
    wav = normalize_volume(resample_to_16k(samples.float().flatten(), src_rate))
    if wav.numel() <= N_FFT // 2:
        return torch.zeros(0, N_MELS)
    spec = torch.stft(wav, N_FFT, HOP, window=hann_window(N_FFT), center=True, pad_mode="reflect", return_complex=True)
    return (slaney_filterbank(SAMPLE_RATE, N_FFT, N_MELS) @ (spec.abs() ** 2)).t().contiguous()


def lstm_layer(x: torch.Tensor, w_ih, w_hh, b_ih, b_hh) -> torch.Tensor:
    """x [T, in] -> hidden states [T, H] (gates in PyTorch order i, f, g, o; zero initial state)."""
    H = w_hh.shape[1]
    pre = x @ w_ih.t() + b_ih + b_hh                    # the input projection of every step at once
    h, c = torch.zeros(H, dtype=x.dtype, device=x.device), torch.zeros(H, dtype=x.dtype, device=x.device)
    out = []
    for t in range(x.shape[0]):
        g = pre[t] + w_hh @ h
        i, f, gg, o = torch.sigmoid(g[:H]), torch.sigmoid(g[H:2 * H]), torch.tanh(g[2 * H:3 * H]), torch.sigmoid(g[3 * H:])
        c = f * c + i * gg
        h = o * torch.tanh(c)
        out.append(h)
    return torch.stack(out)


def l2_normalize(v: torch.Tensor) -> torch.Tensor:
    n = v.norm()
    return v / n if float(n) > 0 else v


class SpeakerEncoder:
    def __init__(self, weights: dict[str, torch.Tensor], device="cpu"):
        self.device = torch.device(device)
        self.w = {k: v.to(self.device, torch.float32) for k, v in weights.items()}
        for k in ("lstm.weight_ih_l0", "lstm.weight_hh_l2", "proj.weight", "proj.bias"):
            if k not in self.w:
                raise LoadError(f"chatterbox_ve: missing tensor {k}")

    @torch.no_grad()
    def forward_block(self, mel: torch.Tensor) -> torch.Tensor:
        x = mel.to(self.device, torch.float32)
        for k in range(NUM_LAYERS):
            x = lstm_layer(x, self.w[f"lstm.weight_ih_l{k}"], self.w[f"lstm.weight_hh_l{k}"],
                           self.w[f"lstm.bias_ih_l{k}"], self.w[f"lstm.bias_hh_l{k}"])
        return torch.relu(self.w["proj.weight"] @ x[-1] + self.w["proj.bias"])

    def embed_mel_frames(self, mel: torch.Tensor) -> torch.Tensor:
        n, part = mel.shape[0], PARTIALS_N_FRAMES
        if n <= part:
            return l2_normalize(self.forward_block(mel))
        starts = list(range(0, n - part + 1, max(1, part // 2)))
        if starts[-1] != n - part:
            starts.append(n - part)
        acc = sum(self.forward_block(mel[s:s + part]) for s in starts) / len(starts)
        return l2_normalize(acc)


class ChatterboxVoiceEmbedder(VoiceEmbedder):
    ID = "chatterbox_ve"

    def __init__(self, encoder: SpeakerEncoder, backend: str):
        self.encoder, self.backend = encoder, backend

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "chatterbox", self.backend, {"dim": EMBED_DIM, "sample_rate": SAMPLE_RATE})

    def embed(self, audio: AudioTrack) -> list[float]:
        if not audio.samples:
            raise AudioError("chatterbox_ve: empty reference audio")
        mono = to_mono(torch.tensor(audio.samples, dtype=torch.float32), audio.channels)
        mel = wav_to_mel_frames(mono, audio.sample_rate)
        if mel.shape[0] == 0:
            raise AudioError("chatterbox_ve: reference audio is too short")
        return self.encoder.embed_mel_frames(mel).cpu().tolist()


def cosine_similarity(a, b) -> float:
    x, y = torch.as_tensor(a, dtype=torch.float32), torch.as_tensor(b, dtype=torch.float32)
    d = float(x.norm() * y.norm())
    return float(x @ y) / d if d > 0 else 0.0
