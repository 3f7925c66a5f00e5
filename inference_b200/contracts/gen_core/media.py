"""Host media buffers that cross the generator contract (gen-core/src/media.rs): images are raw RGB8."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Image:
    width: int
    height: int
    pixels: bytes  # RGB8, row-major

    def __post_init__(self):
        if len(self.pixels) != self.width * self.height * 3:
            raise ValueError(f"Image {self.width}x{self.height} needs {self.width * self.height * 3} RGB bytes")

    def to_ppm(self) -> bytes:
        return f"P6\n{self.width} {self.height}\n255\n".encode() + self.pixels


@dataclass
class AudioTrack:
    sample_rate: int
    channels: int
    samples: list[float] = field(default_factory=list)  # interleaved f32 PCM in [-1, 1]


@dataclass
class AudioChunk:
    """One block of a streamed track: chunks arrive in `index` order and concatenate to the returned track."""
    sample_rate: int
    channels: int
    samples: list[float] = field(default_factory=list)
    index: int = 0
