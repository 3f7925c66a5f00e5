"""Mel filterbanks (candle-audio/src/mel.rs; Whisper's frontend uses the Slaney-normalised variant).

`MelFilterbank` is the HTK-scale triangular bank of the audio commons: unnormalised triangles between n_mels + 2
edges equally spaced in mel, applied to a bin-major spectrum. `slaney_filterbank` is the area-normalised Slaney
scale bank (linear below 1 kHz, logarithmic above) that Whisper's 80-bin front end was trained with."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .dsp import AudioError


def hz_to_mel(hz: float) -> float:
    return 2595.0 * math.log10(1.0 + hz / 700.0)


def mel_to_hz(mel: float) -> float:
    return 700.0 * (10.0 ** (mel / 2595.0) - 1.0)


@dataclass
class MelFilterbank:
    n_mels: int
    n_bins: int
    weights: torch.Tensor       # [n_mels, n_bins]

    @classmethod
    def new(cls, sample_rate: int, n_fft: int, n_mels: int, fmin: float, fmax: float) -> "MelFilterbank":
        if sample_rate == 0 or n_fft < 2 or n_mels == 0:
            raise AudioError("mel filterbank needs sample_rate >= 1, n_fft >= 2, n_mels >= 1 "
                             f"(got {sample_rate}, {n_fft}, {n_mels})")
        nyq = sample_rate / 2.0
        if not (0.0 <= fmin < nyq) or fmax <= fmin or fmax > nyq:
            raise AudioError(f"mel filterbank needs 0 <= fmin < fmax <= nyquist ({nyq} Hz), got fmin={fmin} fmax={fmax}")
        n_bins = n_fft // 2 + 1
        lo, hi = hz_to_mel(fmin), hz_to_mel(fmax)
        edges = torch.tensor([mel_to_hz(lo + (hi - lo) * i / (n_mels + 1)) for i in range(n_mels + 2)])
        f = torch.arange(n_bins, dtype=torch.float32) * sample_rate / n_fft
        left, center, right = edges[:-2, None], edges[1:-1, None], edges[2:, None]
        up, down = (f - left) / (center - left), (right - f) / (right - center)
        w = torch.where(f <= center, up, down)
        w = torch.where((f <= left) | (f >= right), torch.zeros_like(w), w)
        return cls(n_mels, n_bins, w.float())

    def apply(self, spectrum: torch.Tensor, n_frames: int) -> torch.Tensor:
        if spectrum.numel() != self.n_bins * n_frames:
            raise AudioError(f"mel apply expects bin-major [{self.n_bins}, {n_frames}] input "
                             f"({self.n_bins * n_frames} values), got {spectrum.numel()}")
        return self.weights.to(spectrum.device) @ spectrum.reshape(self.n_bins, n_frames).float()


def _slaney_hz_to_mel(f: torch.Tensor) -> torch.Tensor:
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return torch.where(f >= min_log_hz, min_log_mel + torch.log(f.clamp(min=1e-10) / min_log_hz) / logstep, f / f_sp)


def _slaney_mel_to_hz(m: torch.Tensor) -> torch.Tensor:
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return torch.where(m >= min_log_mel, min_log_hz * torch.exp(logstep * (m - min_log_mel)), f_sp * m)


def slaney_filterbank(sample_rate: int, n_fft: int, n_mels: int, fmin: float = 0.0, fmax: float | None = None
                      ) -> torch.Tensor:
    """[n_mels, n_fft / 2 + 1] float32, each triangle scaled by 2 / (its bandwidth in Hz)."""
    fmax = sample_rate / 2.0 if fmax is None else fmax
    d = torch.float64
    fft_f = torch.linspace(0, sample_rate / 2, n_fft // 2 + 1, dtype=d)
    mels = torch.linspace(float(_slaney_hz_to_mel(torch.tensor(fmin, dtype=d))),
                          float(_slaney_hz_to_mel(torch.tensor(fmax, dtype=d))), n_mels + 2, dtype=d)
    hz = _slaney_mel_to_hz(mels)
    fdiff = hz[1:] - hz[:-1]
    ramps = hz[:, None] - fft_f[None, :]
    lower, upper = -ramps[:-2] / fdiff[:-1, None], ramps[2:] / fdiff[1:, None]
    w = torch.clamp(torch.minimum(lower, upper), min=0)
    return (w * (2.0 / (hz[2:] - hz[:-2]))[:, None]).float()
