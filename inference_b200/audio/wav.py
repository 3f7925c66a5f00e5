"""16-bit PCM WAV encode / decode for `AudioTrack` (candle-audio/src/wav.rs)."""
from __future__ import annotations

import struct
from pathlib import Path

from ..contracts.gen_core.media import AudioTrack
from .dsp import AudioError


def encode_wav_pcm16(track: AudioTrack) -> bytes:
    """Canonical 44-byte RIFF header + interleaved little-endian samples: clamp to [-1, 1], scale by 32767,
    truncate toward zero."""
    if track.channels == 0 or track.sample_rate == 0:
        raise AudioError(f"WAV encode needs channels >= 1 and sample_rate >= 1 (got {track.channels} ch @ "
                         f"{track.sample_rate} Hz)")
    n = len(track.samples)
    if n % track.channels != 0:
        raise AudioError(f"WAV encode: {n} samples do not divide into {track.channels} interleaved channels")
    data_len = n * 2
    if data_len > 0xFFFFFFFF - 36:
        raise AudioError(f"WAV encode: {n} samples exceed the 32-bit RIFF size field")
    head = b"RIFF" + struct.pack("<I", 36 + data_len) + b"WAVEfmt " + struct.pack(
        "<IHHIIHH", 16, 1, track.channels, track.sample_rate, track.sample_rate * track.channels * 2,
        track.channels * 2, 16) + b"data" + struct.pack("<I", data_len)
    ints = [int(max(-1.0, min(1.0, s)) * 32767) for s in track.samples]
    return head + struct.pack(f"<{n}h", *ints)


def write_wav_pcm16(path: str | Path, track: AudioTrack) -> None:
    try:
        Path(path).write_bytes(encode_wav_pcm16(track))
    except OSError as e:
        raise AudioError(f"write WAV {path}: {e}") from e


def decode_wav_pcm16(data: bytes) -> AudioTrack:
    """Reads a PCM16 RIFF file (any chunk order; extra chunks are skipped)."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise AudioError("not a RIFF/WAVE file")
    pos, fmt, pcm = 12, None, None
    while pos + 8 <= len(data):
        cid, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
        body = data[pos + 8:pos + 8 + size]
        if cid == b"fmt ":
            fmt = struct.unpack("<HHIIHH", body[:16])
        elif cid == b"data":
            pcm = body
        pos += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise AudioError("WAV file lacks a fmt or data chunk")
    if fmt[0] != 1 or fmt[5] != 16:
        raise AudioError(f"only 16-bit PCM is supported (format {fmt[0]}, {fmt[5]} bits)")
    n = len(pcm) // 2
    return AudioTrack(sample_rate=fmt[2], channels=fmt[1],
                      samples=[v / 32767.0 for v in struct.unpack(f"<{n}h", pcm[:n * 2])])
