"""Audio host math (gen-core/src/audio_dsp.rs:153,303): ITU-R BS.1770-4 integrated loudness (K-weighting, 400 ms
blocks with 75 % overlap, absolute -70 LUFS and relative -10 LU gates), gain to a target loudness, and channel
mixdown."""
from __future__ import annotations

import math

import numpy as np

from .media import AudioTrack


def _biquad(x: np.ndarray, b, a) -> np.ndarray:
    y = np.zeros_like(x)
    x1 = x2 = y1 = y2 = 0.0
    b0, b1, b2 = b
    _, a1, a2 = a
    for i, v in enumerate(x):
        o = b0 * v + b1 * x1 + b2 * x2 - a1 * y1 - a2 * y2
        x2, x1, y2, y1 = x1, v, y1, o
        y[i] = o
    return y


def _k_weighting(fs: float):
    """The two-stage K filter re-derived for any sample rate (coefficients equal the standard's table at 48 kHz)."""
    f0, g, q = 1681.974450955533, 3.999843853973347, 0.7071752369554196
    k = math.tan(math.pi * f0 / fs)
    vh, vb = 10 ** (g / 20), (10 ** (g / 20)) ** 0.4996667741545416
    a0 = 1 + k / q + k * k
    shelf = ([(vh + vb * k / q + k * k) / a0, 2 * (k * k - vh) / a0, (vh - vb * k / q + k * k) / a0],
             [1.0, 2 * (k * k - 1) / a0, (1 - k / q + k * k) / a0])
    f0, q = 38.13547087602444, 0.5003270373238773
    k = math.tan(math.pi * f0 / fs)
    a0 = 1 + k / q + k * k
    hp = ([1.0, -2.0, 1.0], [1.0, 2 * (k * k - 1) / a0, (1 - k / q + k * k) / a0])
    return shelf, hp


def integrated_loudness(track: AudioTrack) -> float:
    """LUFS of the whole track; -inf for silence or clips shorter than one 400 ms block."""
    fs, ch = track.sample_rate, track.channels
    x = np.asarray(track.samples, dtype=np.float64).reshape(-1, ch)
    shelf, hp = _k_weighting(fs)
    block, hop = int(0.4 * fs), int(0.1 * fs)
    if x.shape[0] < block:
        return float("-inf")
    weights = [1.0, 1.0, 1.0, 0.0, 1.41, 1.41][:ch] if ch <= 6 else [1.0] * ch   # L R C LFE Ls Rs
    filt = np.stack([_biquad(_biquad(x[:, c], *shelf), *hp) for c in range(ch)], 1)
    z = []
    for s in range(0, x.shape[0] - block + 1, hop):
        z.append(sum(w * float(np.mean(filt[s:s + block, c] ** 2)) for c, w in enumerate(weights)))
    z = np.asarray(z)
    lk = -0.691 + 10 * np.log10(np.maximum(z, 1e-30))
    keep = z[lk > -70.0]
    if keep.size == 0:
        return float("-inf")
    rel = -0.691 + 10 * math.log10(float(keep.mean())) - 10.0
    keep = z[(lk > -70.0) & (lk > rel)]
    if keep.size == 0:
        return float("-inf")
    return -0.691 + 10 * math.log10(float(keep.mean()))


def normalize_loudness(track: AudioTrack, target_lufs: float = -16.0, peak_ceiling: float = 0.98) -> AudioTrack:
    lufs = integrated_loudness(track)
    if not math.isfinite(lufs):
        return track
    gain = 10 ** ((target_lufs - lufs) / 20)
    x = np.asarray(track.samples, dtype=np.float64) * gain
    peak = float(np.max(np.abs(x))) if x.size else 0.0
    if peak > peak_ceiling:
        x *= peak_ceiling / peak
    return AudioTrack(track.sample_rate, track.channels, x.astype(np.float32).tolist())


def mixdown_mono(track: AudioTrack) -> AudioTrack:
    if track.channels == 1:
        return track
    x = np.asarray(track.samples, dtype=np.float32).reshape(-1, track.channels).mean(1)
    return AudioTrack(track.sample_rate, 1, x.tolist())
