"""Whisper speech recognition: log-mel front end, encoder-decoder transformer, windowed decoding into timed segments
(the reference's candle-audio-whisper crate: src/mel.rs, src/model.rs, src/decode.rs).

Weights use the Hugging Face `WhisperForConditionalGeneration` key names. On a CUDA device the model runs in bf16
with every projection on the tcgen05 GEMM (`ops.linear`, bias fused in its epilogue); the decoder keeps a per-layer
self-attention K/V cache and computes each layer's cross-attention K/V once per 30-second window. On the CPU the same
code runs in fp32 and is the oracle the tests compare against the Hugging Face implementation."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Protocol

import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, LoadError
from ..contracts.gen_core.media import AudioTrack
from ..contracts.gen_core.traits import SimpleDescriptor, Transcriber, TranscriptSegment
from .dsp import AudioError, hann_window
from .mel import slaney_filterbank

SAMPLE_RATE = 16_000
N_FFT = 400
HOP_LENGTH = 160
CHUNK_SECONDS = 30
N_SAMPLES = CHUNK_SECONDS * SAMPLE_RATE
N_FRAMES = N_SAMPLES // HOP_LENGTH          # 3000 mel frames per window

LANGUAGES = ("en zh de es ru ko fr ja pt tr pl ca nl ar sv it id hi fi vi he uk el ms cs ro da hu ta no th ur hr bg lt "
             "la mi ml cy sk te fa lv bn sr az sl kn et mk br eu is hy ne mn bs kk sq sw gl mr pa si km sn yo so af oc "
             "ka be tg sd gu am yi lo uz fo ht ps tk nn mt sa lb my bo tl mg as tt haw ln ha ba jw su").split()


@dataclass
class WhisperConfig:
    vocab_size: int = 51865
    num_mel_bins: int = 80
    d_model: int = 384
    encoder_layers: int = 4
    encoder_attention_heads: int = 6
    decoder_layers: int = 4
    decoder_attention_heads: int = 6
    encoder_ffn_dim: int = 1536
    decoder_ffn_dim: int = 1536
    max_source_positions: int = 1500
    max_target_positions: int = 448
    suppress_tokens: list[int] = field(default_factory=list)

    @classmethod
    def from_json(cls, d: dict) -> "WhisperConfig":
        keys = cls.__dataclass_fields__.keys()
        return cls(**{k: (d[k] if d[k] is not None else []) if k == "suppress_tokens" else d[k] for k in keys if k in d})


# ---- front end ---------------------------------------------------------------------------------------------------------
def to_mono(samples: torch.Tensor, channels: int) -> torch.Tensor:
    return samples if channels <= 1 else samples.reshape(-1, channels).mean(dim=1)


def resample_to_16k(samples: torch.Tensor, src_rate: int) -> torch.Tensor:
    """Linear interpolation to 16 kHz (the reference's resampler; adequate for speech front ends)."""
    if src_rate == SAMPLE_RATE or samples.numel() == 0:
        return samples
    ratio = SAMPLE_RATE / src_rate
    out_len = int(round(samples.numel() * ratio))
    pos = torch.arange(out_len, dtype=torch.float64) / ratio
    left = pos.floor().long()
    frac = (pos - left).float()
    last = samples.numel() - 1
    a, b = samples[left.clamp(max=last)], samples[(left + 1).clamp(max=last)]
    return a + (b - a) * frac


def log_mel_spectrogram(pcm: torch.Tensor, n_mels: int = 80, pad_to_window: bool = True) -> torch.Tensor:
    """[n_mels, frames] Whisper features: 25 ms periodic-Hann frames every 10 ms, power spectrum, Slaney mel bank,
    log10 clamped to 8 orders of magnitude below the peak, then (x + 4) / 4. With pad_to_window the audio is
    zero-padded to a whole number of 30-second windows."""
    pcm = pcm.float().flatten()
    if pad_to_window:
        n = max(1, math.ceil(pcm.numel() / N_SAMPLES)) * N_SAMPLES
        pcm = F.pad(pcm, (0, n - pcm.numel()))
    spec = torch.stft(pcm, N_FFT, HOP_LENGTH, window=hann_window(N_FFT).to(pcm.device), center=True,
                      pad_mode="reflect", return_complex=True)
    power = spec[:, :-1].abs() ** 2
    mel = slaney_filterbank(SAMPLE_RATE, N_FFT, n_mels).to(pcm.device) @ power
    log = torch.log10(mel.clamp(min=1e-10))
    log = torch.maximum(log, log.max() - 8.0)
    return (log + 4.0) / 4.0


def track_to_mel(track: AudioTrack, n_mels: int = 80) -> torch.Tensor:
    pcm = resample_to_16k(to_mono(torch.tensor(track.samples, dtype=torch.float32), track.channels), track.sample_rate)
    return log_mel_spectrogram(pcm, n_mels)


def sinusoids(length: int, channels: int) -> torch.Tensor:
    inc = math.log(10000.0) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)


# ---- model ---------------------------------------------------------------------------------------------------------------
class WhisperModel:
    def __init__(self, cfg: WhisperConfig, weights: dict[str, torch.Tensor], device: str | torch.device = "cpu",
                 dtype: torch.dtype | None = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        strip = lambda k: k[len("model."):] if k.startswith("model.") else k
        self.w = {strip(k): v.to(self.device, self.dtype) for k, v in weights.items() if v.is_floating_point()}
        for need in ("encoder.conv1.weight", "decoder.embed_tokens.weight", "decoder.embed_positions.weight"):
            if need not in self.w:
                raise LoadError(f"whisper: missing tensor {need}")
        if "encoder.embed_positions.weight" not in self.w:
            self.w["encoder.embed_positions.weight"] = sinusoids(cfg.max_source_positions, cfg.d_model).to(
                self.device, self.dtype)
        self._self_kv: list[tuple[torch.Tensor, torch.Tensor] | None] = []
        self._cross_kv: list[tuple[torch.Tensor, torch.Tensor]] = []

    # projections: tcgen05 GEMM with the bias in its epilogue on a GPU, plain matmul on the CPU
    def _lin(self, x: torch.Tensor, name: str, act: str | None = None) -> torch.Tensor:
        w, b = self.w[name + ".weight"], self.w.get(name + ".bias")
        if x.is_cuda and x.dtype == torch.bfloat16 and w.shape[1] % 8 == 0:
            from ..ops import linear

            y = linear(x.contiguous(), w, b)
        else:
            y = F.linear(x, w, b)
        return F.gelu(y) if act == "gelu" else y

    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.layer_norm(x, (x.shape[-1],), self.w[name + ".weight"], self.w[name + ".bias"], 1e-5)

    def _heads(self, x: torch.Tensor, n: int) -> torch.Tensor:
        b, t, d = x.shape
        return x.view(b, t, n, d // n).transpose(1, 2)

    def _attn(self, q, k, v, n_heads: int, causal: bool) -> torch.Tensor:
        o = F.scaled_dot_product_attention(self._heads(q, n_heads), k, v, is_causal=causal and q.shape[1] > 1)
        return o.transpose(1, 2).reshape(q.shape)

    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [B, n_mels, frames <= 2 * max_source_positions] -> [B, frames / 2, d_model]."""
        c = self.cfg
        x = mel.to(self.device, self.dtype)
        x = F.gelu(F.conv1d(x, self.w["encoder.conv1.weight"], self.w["encoder.conv1.bias"], padding=1))
        x = F.gelu(F.conv1d(x, self.w["encoder.conv2.weight"], self.w["encoder.conv2.bias"], stride=2, padding=1))
        x = x.transpose(1, 2)
        x = x + self.w["encoder.embed_positions.weight"][: x.shape[1]]
        H = c.encoder_attention_heads
        for i in range(c.encoder_layers):
            p = f"encoder.layers.{i}"
            h = self._ln(x, p + ".self_attn_layer_norm")
            q, k, v = (self._lin(h, f"{p}.self_attn.{n}_proj") for n in "qkv")
            x = x + self._lin(self._attn(q, self._heads(k, H), self._heads(v, H), H, False), p + ".self_attn.out_proj")
            h = self._ln(x, p + ".final_layer_norm")
            x = x + self._lin(self._lin(h, p + ".fc1", act="gelu"), p + ".fc2")
        return self._ln(x, "encoder.layer_norm")

    def reset_kv_cache(self) -> None:
        self._self_kv, self._cross_kv = [], []

    def decode(self, tokens: torch.Tensor, audio: torch.Tensor, flush: bool) -> torch.Tensor:
        """Decoder hidden states [B, T, d_model] for ALL of `tokens` [B, T]: with flush the caches are rebuilt from
        the whole sequence; otherwise only the positions beyond the cached length are computed."""
        c = self.cfg
        H = c.decoder_attention_heads
        if flush:
            self.reset_kv_cache()
        past = self._self_kv[0][0].shape[2] if self._self_kv and self._self_kv[0] is not None else 0
        new = tokens[:, past:].to(self.device)
        x = self.w["decoder.embed_tokens.weight"][new] + \
            self.w["decoder.embed_positions.weight"][past:past + new.shape[1]]
        first = not self._cross_kv
        if not self._self_kv:
            self._self_kv = [None] * c.decoder_layers
        for i in range(c.decoder_layers):
            p = f"decoder.layers.{i}"
            h = self._ln(x, p + ".self_attn_layer_norm")
            q, k, v = (self._lin(h, f"{p}.self_attn.{n}_proj") for n in "qkv")
            k, v = self._heads(k, H), self._heads(v, H)
            if self._self_kv[i] is not None:
                k, v = torch.cat([self._self_kv[i][0], k], dim=2), torch.cat([self._self_kv[i][1], v], dim=2)
            self._self_kv[i] = (k, v)
            if past == 0:
                a = self._attn(q, k, v, H, True)
            else:       # new rows attend to everything cached plus, causally, to each other
                T, S = q.shape[1], k.shape[2]
                mask = torch.ones(T, S, dtype=torch.bool, device=q.device).tril(diagonal=S - T)
                a = F.scaled_dot_product_attention(self._heads(q, H), k, v, attn_mask=mask).transpose(1, 2).reshape(
                    q.shape)
            x = x + self._lin(a, p + ".self_attn.out_proj")
            h = self._ln(x, p + ".encoder_attn_layer_norm")
            if first:
                self._cross_kv.append((self._heads(self._lin(audio, p + ".encoder_attn.k_proj"), H),
                                       self._heads(self._lin(audio, p + ".encoder_attn.v_proj"), H)))
            ck, cv = self._cross_kv[i]
            x = x + self._lin(self._attn(self._lin(h, p + ".encoder_attn.q_proj"), ck, cv, H, False),
                              p + ".encoder_attn.out_proj")
            h = self._ln(x, p + ".final_layer_norm")
            x = x + self._lin(self._lin(h, p + ".fc1", act="gelu"), p + ".fc2")
        return self._ln(x, "decoder.layer_norm")

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        w = self.w.get("proj_out.weight", self.w["decoder.embed_tokens.weight"])
        return (hidden.float() @ w.float().t()) if not hidden.is_cuda else F.linear(hidden, w).float()


# ---- decoding ------------------------------------------------------------------------------------------------------------
class TokenizerLike(Protocol):
    def token_to_id(self, token: str) -> int | None: ...
    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str: ...


@dataclass
class DecodeOutput:
    text: str
    segments: list[TranscriptSegment]
    tokens: int
    finish_reason: str          # "stop_token" | "max_tokens"


def token_id(tok: TokenizerLike, token: str) -> int:
    i = tok.token_to_id(token)
    if i is None:
        raise AudioError(f"whisper: tokenizer has no id for {token!r}")
    return i


class WhisperDecoder:
    def __init__(self, model: WhisperModel, tokenizer: TokenizerLike, timestamps: bool):
        self.model, self.tok = model, tokenizer
        self.sot, self.eot = token_id(tokenizer, "<|startoftranscript|>"), token_id(tokenizer, "<|endoftext|>")
        self.transcribe_token = token_id(tokenizer, "<|transcribe|>")
        self.translate_token = token_id(tokenizer, "<|translate|>")
        self.no_timestamps = token_id(tokenizer, "<|notimestamps|>")
        sup = torch.zeros(model.cfg.vocab_size)
        for i in model.cfg.suppress_tokens:
            if 0 <= i < model.cfg.vocab_size:
                sup[i] = float("-inf")
        if timestamps:
            sup[self.no_timestamps] = float("-inf")
        self.suppress = sup.to(model.device)

    def language_token(self, code: str) -> int:
        if code not in LANGUAGES:
            raise AudioError(f"whisper: language {code!r} is not a Whisper language code")
        return token_id(self.tok, f"<|{code}|>")

    def detect_language(self, mel: torch.Tensor) -> int:
        """The language token with the highest probability after the start-of-transcript token."""
        ids = [i for i in (self.tok.token_to_id(f"<|{c}|>") for c in LANGUAGES) if i is not None]
        m = self.model
        audio = m.encode(mel[:, :, : 2 * m.cfg.max_source_positions])
        h = m.decode(torch.tensor([[self.sot]]), audio, True)
        lg = m.logits(h[:, :1])[0, 0]
        best = int(lg[torch.tensor(ids, device=lg.device)].argmax())
        m.reset_kv_cache()
        return ids[best]

    def timestamp_seconds(self, token: int) -> float | None:
        begin = self.no_timestamps + 1
        return (token - begin) * 0.02 if token >= begin else None

    def decode_window(self, mel, language_token, translate, timestamps, temperature, seed, max_new_tokens,
                      cancel: Callable[[], bool]) -> tuple[list[int], bool]:
        m = self.model
        audio = m.encode(mel)
        gen = torch.Generator().manual_seed(seed)
        tokens = [self.sot] + ([language_token] if language_token is not None else [])
        tokens.append(self.translate_token if translate else self.transcribe_token)
        if not timestamps:
            tokens.append(self.no_timestamps)
        prompt_len = len(tokens)
        hit_eot = False
        for i in range(min(max_new_tokens, m.cfg.max_target_positions)):
            if cancel():
                raise Canceled()
            h = m.decode(torch.tensor([tokens]), audio, i == 0)
            lg = m.logits(h[:, -1:])[0, 0] + self.suppress
            if temperature > 0:
                nxt = int(torch.multinomial(torch.softmax(lg.cpu() / temperature, -1), 1, generator=gen))
            else:
                nxt = int(lg.argmax())
            tokens.append(nxt)
            if nxt == self.eot or len(tokens) > m.cfg.max_target_positions:
                hit_eot = nxt == self.eot
                break
        m.reset_kv_cache()
        return tokens[prompt_len:], hit_eot

    def run(self, mel: torch.Tensor, language_token: int | None = None, translate: bool = False,
            timestamps: bool = True, temperature: float = 0.0, seed: int = 0, max_new_tokens: int = 224,
            cancel: Callable[[], bool] = lambda: False) -> DecodeOutput:
        """Walks the features in 30-second windows; each window decodes independently."""
        frames = mel.shape[2]
        seek, texts, segments, total, finish = 0, [], [], 0, "stop_token"
        while seek < frames:
            size = min(frames - seek, N_FRAMES)
            toks, hit = self.decode_window(mel[:, :, seek:seek + size], language_token, translate, timestamps,
                                           temperature, seed, max_new_tokens, cancel)
            total += len(toks)
            if not hit:
                finish = "max_tokens"
            self._append_window(toks, seek * HOP_LENGTH / SAMPLE_RATE, timestamps, texts, segments)
            seek += size
        return DecodeOutput(" ".join(texts).strip(), segments, total, finish)

    def _append_window(self, toks, offset: float, timestamps: bool, texts: list[str],
                       segments: list[TranscriptSegment]) -> None:
        if not timestamps:
            t = self.tok.decode(toks, True).strip()
            if t:
                texts.append(t)
            return
        pending: list[int] = []
        start = offset

        def flush(end: float) -> None:
            t = self.tok.decode(pending, True).strip()
            if t:
                segments.append(TranscriptSegment(start=start, end=end, text=t))
                texts.append(t)
            pending.clear()
        for tk in toks:
            if tk in (self.sot, self.eot):
                continue
            ts = self.timestamp_seconds(tk)
            if ts is None:
                pending.append(tk)
                continue
            if pending:
                flush(offset + ts)
            start = offset + ts
        if pending:
            flush(start)


class WhisperTranscriber(Transcriber):
    """`Transcriber` provider over a Hugging Face Whisper snapshot directory (config.json, tokenizer.json,
    model.safetensors)."""

    ID = "whisper"

    def __init__(self, model: WhisperModel, tokenizer: TokenizerLike, backend: str):
        self.model, self.tok, self.backend = model, tokenizer, backend

    @classmethod
    def load_dir(cls, path, device="cpu", backend: str = "cpu") -> "WhisperTranscriber":
        import json
        from pathlib import Path

        from ..contracts.core_llm.tokenizer import Tokenizer
        from ..io.safetensors_io import load_dir

        p = Path(path)
        cfg = WhisperConfig.from_json(json.loads((p / "config.json").read_text()))
        if cfg.num_mel_bins != 80:
            raise LoadError(f"whisper: no mel filterbank for num_mel_bins={cfg.num_mel_bins} (80-bin models only)")
        return cls(WhisperModel(cfg, load_dir(p), device), Tokenizer.from_file(p / "tokenizer.json"), backend)

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "whisper", self.backend, {"sample_rate": SAMPLE_RATE, "window_s": CHUNK_SECONDS})

    def transcribe_full(self, audio: AudioTrack, language: str | None = None, translate: bool = False,
                        timestamps: bool = True, temperature: float = 0.0, seed: int = 0,
                        max_new_tokens: int = 224, cancel: Callable[[], bool] = lambda: False) -> DecodeOutput:
        if not audio.samples:
            raise AudioError("whisper: empty audio")
        mel = track_to_mel(audio, self.model.cfg.num_mel_bins).unsqueeze(0)
        dec = WhisperDecoder(self.model, self.tok, timestamps)
        lang = dec.language_token(language) if language else dec.detect_language(mel)
        return dec.run(mel, lang, translate, timestamps, temperature, seed, max_new_tokens, cancel)

    def transcribe(self, audio: AudioTrack, language: str | None = None) -> list[TranscriptSegment]:
        return self.transcribe_full(audio, language).segments
