"""Audio family: signal-processing commons, WAV IO, and the model providers (Whisper transcriber, CLAP-style audio
embedder) registered by `audio.catalog` (the reference's candle-audio lane, crates/audio/*)."""
from .dsp import Spectrogram, hann_window, istft, stft  # noqa: F401
from .mel import MelFilterbank  # noqa: F401
from .wav import decode_wav_pcm16, encode_wav_pcm16, write_wav_pcm16  # noqa: F401
