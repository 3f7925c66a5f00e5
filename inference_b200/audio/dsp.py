"""STFT / inverse STFT commons (candle-audio/src/dsp.rs).

Conventions: periodic Hann window; centred frames with reflect padding of n_fft / 2 on both sides; n_fft a power of
two; spectra stored bin-major [n_bins, n_frames]; the inverse overlap-adds windowed frames, divides by the summed
squared window and trims the padding. The transforms run as batched torch FFTs over all frames at once."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


class AudioError(Exception):
    pass


def hann_window(length: int) -> torch.Tensor:
    i = torch.arange(length, dtype=torch.float32)
    return 0.5 * (1.0 - torch.cos(2.0 * math.pi * i / length))


@dataclass
class Spectrogram:
    n_bins: int
    n_frames: int
    re: torch.Tensor        # [n_bins, n_frames]
    im: torch.Tensor

    def magnitude(self) -> torch.Tensor:
        return torch.sqrt(self.re * self.re + self.im * self.im)

    def phase(self) -> torch.Tensor:
        return torch.atan2(self.im, self.re)


def _require(n_fft: int, hop: int, window: torch.Tensor) -> None:
    if n_fft < 2 or n_fft & (n_fft - 1):
        raise AudioError(f"n_fft {n_fft} must be a power of two >= 2 (radix-2 STFT)")
    if window.numel() != n_fft:
        raise AudioError(f"window length {window.numel()} does not match n_fft {n_fft}")
    if hop == 0:
        raise AudioError("hop must be >= 1")


def stft(samples: torch.Tensor, n_fft: int, hop: int, window: torch.Tensor) -> Spectrogram:
    samples = torch.as_tensor(samples, dtype=torch.float32).flatten()
    _require(n_fft, hop, window)
    n = samples.numel()
    if n < 2:
        raise AudioError(f"stft needs at least 2 samples to reflect-pad, got {n}")
    pad = n_fft // 2
    if pad >= n:
        raise AudioError(f"stft reflect pad {pad} needs input longer than n_fft/2, got {n} samples")
    padded = torch.cat([samples[1:pad + 1].flip(0), samples, samples[n - 1 - pad:n - 1].flip(0)])
    frames = padded.unfold(0, n_fft, hop) * window.to(samples.device)
    spec = torch.fft.rfft(frames, dim=-1).t()
    return Spectrogram(n_fft // 2 + 1, frames.shape[0], spec.real.contiguous(), spec.imag.contiguous())


def istft(magnitude: torch.Tensor, phase: torch.Tensor, n_frames: int, n_fft: int, hop: int,
          window: torch.Tensor) -> torch.Tensor:
    _require(n_fft, hop, window)
    n_bins = n_fft // 2 + 1
    if magnitude.numel() != n_bins * n_frames or phase.numel() != n_bins * n_frames:
        raise AudioError(f"istft expects bin-major [{n_bins}, {n_frames}] magnitude and phase "
                         f"({n_bins * n_frames} values), got {magnitude.numel()} and {phase.numel()}")
    if n_frames == 0:
        return torch.zeros(0)
    m, p = magnitude.reshape(n_bins, n_frames).float(), phase.reshape(n_bins, n_frames).float()
    frames = torch.fft.irfft(torch.complex(m * torch.cos(p), m * torch.sin(p)).t(), n=n_fft, dim=-1)
    w = window.to(frames.device)
    out_len = n_fft + (n_frames - 1) * hop
    idx = (torch.arange(n_frames, device=frames.device).unsqueeze(1) * hop
           + torch.arange(n_fft, device=frames.device).unsqueeze(0)).reshape(-1)
    out = torch.zeros(out_len, device=frames.device).index_add_(0, idx, (frames * w).reshape(-1))
    wsum = torch.zeros(out_len, device=frames.device).index_add_(0, idx, (w * w).expand(n_frames, -1).reshape(-1))
    out = torch.where(wsum > 1e-8, out / wsum.clamp(min=1e-8), out)
    pad = n_fft // 2
    end = max(out_len - pad, 0)
    return out[min(pad, end):end]


def nearest_upsample1d(x: torch.Tensor, k: int) -> torch.Tensor:
    """[B, C, T] -> [B, C, T * k], each frame repeated k times (candle-audio/src/ops.rs)."""
    b, c, t = x.shape
    return x.unsqueeze(3).expand(b, c, t, k).reshape(b, c, t * k)
