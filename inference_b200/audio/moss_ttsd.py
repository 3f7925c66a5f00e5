"""MOSS-TTSD multi-speaker dialogue text-to-speech `moss_ttsd_v05` (parity: candle-audio-moss-tts/src/{config,backbone,
decode,sampling,codec,model}.rs).

A delay-pattern autoregressive model over residual-VQ speech codes. Every position is an 8-channel token: channel 0 is
a text / speech id of the language model's vocabulary (which also carries codebook 0 as a range of ids), channels 1..7
the remaining codebooks; each channel has its own embedding table, the eight embeddings are summed, a Qwen3 decoder runs
on the sum, and each channel's logits are the final-norm state times that channel's (tied) embedding table. Channel j
is delayed by j positions: the prompt grid is shifted, generation teacher-forces the shifted prompt tail, samples every
channel at every position (temperature 0.9, top-k 50, top-p 0.95, a seeded SplitMix64 stream), and after the text
channel leaves the speech range the remaining channels are drained for seven more positions. Un-shifting yields clean
frames at 12.5 Hz.

The codes are rendered by the XY_Tokenizer codec (a separate checkpoint, passed in as the `codec` component): the eight
codebook vectors are summed and projected to 3072 channels, a 4-layer full-attention adapter, a x4 transposed convolution
(50 Hz), a 12-layer acoustic transformer with two transposed convolutions (80 mel bins at 100 Hz), a 30-block ConvNeXt
vocoder whose head predicts log-magnitude and phase, and an inverse STFT (size 960, hop 240, Hann overlap-add with
window-envelope normalisation): 1920 samples per frame at 24 kHz.

Backends: the decoder runs through this package's reference decoder (`OracleLlama`, a growing key / value cache; fp32 on
CPU, bf16 tensor ops on a CUDA device) because its inputs are summed embeddings, not token ids; the codec runs in fp32."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, GenerationOutput, GenerationRequest, Generator, Modality,
                                            ModelDescriptor)
from ..contracts.gen_core.license import WeightLicense
from ..contracts.gen_core.media import AudioTrack
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec, ProgressDecoding, ProgressStep
from ..contracts.gen_core.traits import reject_unknown_components, require_component

MODEL_ID, FAMILY, SAMPLE_RATE, FRAME_RATE_HZ, SAMPLES_PER_FRAME = "moss_ttsd_v05", "moss_ttsd", 24_000, 12.5, 1920
MAX_DURATION_SECS, DEFAULT_SECONDS, DEFAULT_SAMPLING_SEED, MAX_SPEAKERS = 300.0, 10.0, 13_360, 2
CODEC_COMPONENT_ID, CODEC_CHECKPOINT_FILE, MODEL_WEIGHTS = "codec", "xy_tokenizer.ckpt", "model.safetensors"
LANGUAGES = ["zh", "en", "de", "es", "fr", "ja", "it", "he", "ko", "ru", "fa", "ar", "pl", "pt", "cs", "da", "sv", "hu", "el", "tr"]
DEFAULT_SYSTEM_PROMPT = ("You are a speech synthesizer that generates natural, realistic, and human-like conversational audio "
                         "from dialogue text.")
TEMPERATURE, TOP_P, TOP_K = 0.9, 0.95, 50
MOSS_TTSD_LICENSE = WeightLicense("Apache-2.0", "Apache License 2.0", "https://huggingface.co/OpenMOSS-Team/MOSS-TTSD-v0.5",
                                  "MOSS-TTSD-v0.5 (c) OpenMOSS Team - licensed under Apache-2.0", True)
M64 = (1 << 64) - 1


@dataclass
class MossTtsdConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    attention_bias: bool = False
    channels: int = 8
    speech_vocab_size: int = 1025
    speech_pad_token: int = 1024
    speech_token_range: tuple = (151_665, 152_689)
    speech_eos_token: int = 152_694
    text_pad_id: int = 151_643

    @staticmethod
    def from_json(j: dict) -> "MossTtsdConfig":
        if "bos_token_id" in j and "text_pad_id" not in j:
            j = {**j, "text_pad_id": j["bos_token_id"]}
        try:
            c = MossTtsdConfig(**{k: j[k] for k in MossTtsdConfig.__dataclass_fields__ if k in j})
        except TypeError as e:
            raise LoadError(f"parse MOSS-TTSD config.json: {e}") from e
        c.speech_token_range = tuple(c.speech_token_range)
        if c.channels < 2:
            raise LoadError(f"config.json: channels ({c.channels}) must be >= 2 (text + >=1 audio codebook)")
        if c.speech_vocab_size <= 0:
            raise LoadError("config.json: speech_vocab_size must be > 0")
        lo, hi = c.speech_token_range
        if hi <= lo:
            raise LoadError(f"config.json: speech_token_range {list(c.speech_token_range)} is not an increasing [start, end)")
        if hi - lo < c.speech_vocab_size - 1:
            raise LoadError(f"config.json: speech_token_range width {hi - lo} < codebook-0 code count {c.speech_vocab_size - 1}")
        return c


# ---- seeded sampling ------------------------------------------------------------------------------------------------------
class Rng:
    """SplitMix64; next_f32 is the top 24 bits as a fraction in [0, 1)."""

    def __init__(self, seed: int):
        self.state = (seed ^ 0x9E3779B97F4A7C15) & M64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


def sample(logits: torch.Tensor, rng: Rng, temperature: float = TEMPERATURE, top_k: int = TOP_K, top_p: float = TOP_P) -> int:
    """One draw from 1-D fp32 logits: temperature, keep the top_k largest (ties kept), drop the low-probability tail
    whose mass is <= 1 - top_p (never the most likely token), inverse-CDF in index order."""
    n = logits.numel()
    if n == 0:
        return 0
    if temperature <= 0.0:
        return int(torch.argmax(logits))
    lg = logits.float() / temperature
    k = min(max(top_k, 1), n)
    if k < n:
        kth = torch.topk(lg, k).values[-1]
        lg = torch.where(lg < kth, torch.full_like(lg, float("-inf")), lg)
    if 0.0 < top_p < 1.0:
        probs = _softmax(lg)
        order = torch.argsort(lg, stable=True)                       # ascending
        cum = torch.cumsum(probs[order], 0)
        drop = cum <= (1.0 - top_p)
        drop[-1] = False
        lg = lg.clone()
        lg[order[drop]] = float("-inf")
    probs = _softmax(lg)
    u = rng.next_f32()
    cum = torch.cumsum(probs, 0)
    idx = int(torch.searchsorted(cum, torch.tensor(u, dtype=cum.dtype), right=True))
    if idx >= n:
        nz = torch.nonzero(probs > 0)
        return int(nz[-1]) if nz.numel() else 0
    return idx


def _softmax(lg: torch.Tensor) -> torch.Tensor:
    m = lg.max()
    if not torch.isfinite(m):
        return torch.full_like(lg, 1.0 / lg.numel())
    e = torch.exp(lg - m)
    s = e.sum()
    return e / s if s > 0 else e


# ---- prompt grid and the delay pattern ----------------------------------------------------------------------------------------
def format_dialogue_text(text: str) -> str:
    return text.replace("[S1]", "<speaker1>").replace("[S2]", "<speaker2>")


def build_prompt_grid(tokenizer, cfg: MossTtsdConfig, dialogue: str, system_prompt: str = DEFAULT_SYSTEM_PROMPT) -> list[list[int]]:
    prompt = (f"<|begin_of_style|>{system_prompt}<|end_of_style|>\n<|begin_of_text|>{format_dialogue_text(dialogue)}"
              "<|end_of_text|>\n<|begin_of_speech|>")
    ids = tokenizer.encode(prompt, add_special_tokens=False).ids
    if not ids:
        raise InferenceError("empty prompt after tokenization")
    return [[i] + [cfg.speech_pad_token] * (cfg.channels - 1) for i in ids]


def shift_grid(grid: list[list[int]], cfg: MossTtsdConfig) -> list[list[int]]:
    ch = cfg.channels
    out = [[cfg.text_pad_id] + [cfg.speech_pad_token] * (ch - 1) for _ in range(len(grid) + ch - 1)]
    for j in range(ch):
        for r, src in enumerate(grid):
            out[j + r][j] = src[j]
    return out


def unshift(emitted: list[list[int]], cfg: MossTtsdConfig) -> list[list[int]]:
    ch, strip = cfg.channels, cfg.channels - 1
    out = []
    for t in range(max(0, len(emitted) - strip)):
        cb = [emitted[t + j][j] for j in range(ch)]
        if cfg.speech_pad_token in cb[1:]:
            continue
        cb[0] = max(0, cb[0] - cfg.speech_token_range[0])
        out.append(cb)
    return out


class Backbone:
    def __init__(self, cfg: MossTtsdConfig, weights: dict[str, torch.Tensor], device="cpu"):
        from ..models.config import ModelConfig
        from ..models.oracle import OracleLlama

        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        lcfg = ModelConfig.from_json({
            "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            "intermediate_size": cfg.intermediate_size, "num_hidden_layers": cfg.num_hidden_layers,
            "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta, "attention_bias": cfg.attention_bias,
            "tie_word_embeddings": True, "max_position_embeddings": 32768})
        lm = {"model." + k[len("model.language_model."):]: v for k, v in weights.items() if k.startswith("model.language_model.")}
        self.tables = []
        for c in range(cfg.channels):
            k = f"model.embedding_list.{c}.weight"
            if k not in weights:
                raise LoadError(f"{MODEL_ID}: checkpoint lacks {k}")
            self.tables.append(weights[k].to(self.device, self.dtype))
        lm["model.embed_tokens.weight"] = weights["model.embedding_list.0.weight"]
        self.lm = OracleLlama(lcfg, lm, self.dtype, self.device)

    def new_cache(self):
        from ..models.oracle import ContiguousKvCache

        return ContiguousKvCache(self.cfg.num_hidden_layers)

    def embed(self, frames: list[list[int]]) -> torch.Tensor:
        t = torch.tensor(frames, dtype=torch.int64, device=self.device)                # [T, channels]
        return sum(self.tables[c][t[:, c]] for c in range(self.cfg.channels))[None]

    @torch.no_grad()
    def forward(self, frames: list[list[int]], cache) -> torch.Tensor:
        """Append `frames` to the cache; the final-norm state of the last position [hidden]."""
        h = self.lm.hidden_states(None, cache, cache.offset, embeds=self.embed(frames))
        return self.lm._norm(h[:, -1:], "model.norm.weight")[0, 0]

    def channel_logits(self, hidden: torch.Tensor) -> list[torch.Tensor]:
        return [(self.tables[c] @ hidden.to(self.dtype)).float().cpu() for c in range(self.cfg.channels)]


def run_decoder(backbone: Backbone, grid: list[list[int]], max_positions: int, seed: int, cancel=lambda: False,
                on_position=lambda step: None) -> tuple[list[list[int]], str] | None:
    """The delay-pattern loop -> (clean frames, "eos" | "budget"); None when cancelled."""
    cfg = backbone.cfg
    ch, strip = cfg.channels, cfg.channels - 1
    rng = Rng(seed)
    tf = shift_grid(grid, cfg)
    tf_len = len(tf)
    inputs = [list(f) for f in tf[:tf_len - strip]]
    base = len(inputs)
    cache, prefilled, needs_additional, emitted, stop = backbone.new_cache(), False, -1, [], "budget"
    lo, hi = cfg.speech_token_range
    for step in range(max_positions):
        if cancel():
            return None
        hidden = backbone.forward(inputs if not prefilled else inputs[-1:], cache)
        prefilled = True
        logits = backbone.channel_logits(hidden)
        pos = len(inputs)
        nxt = [0] * ch
        for i, lg in enumerate(logits):
            if i != 0:
                if pos >= tf_len - strip + i and cfg.speech_pad_token < lg.numel():
                    lg[cfg.speech_pad_token] = float("-inf")          # the delayed channel has started: no padding
            elif pos < tf_len and cfg.speech_eos_token < lg.numel():
                lg[cfg.speech_eos_token] = float("-inf")              # no end of speech inside the teacher-forced ramp
            nxt[i] = sample(lg, rng)
        if not (lo <= nxt[0] < hi) and needs_additional < 0:
            needs_additional = strip
        if pos < tf_len:
            i0 = pos + 1 - base
            nxt[i0:ch] = tf[pos][i0:ch]
        if 0 < needs_additional < strip:
            nxt[0] = cfg.speech_eos_token
            for c in range(1, ch):
                if needs_additional < ch - c:
                    nxt[c] = cfg.speech_pad_token
        inputs.append(list(nxt))
        emitted.append(list(nxt))
        if needs_additional > 0:
            needs_additional -= 1
        if needs_additional == 0:
            stop = "eos"
            break
        on_position(step)
    return unshift(emitted, cfg), stop


# ---- XY_Tokenizer codec (decode side) ------------------------------------------------------------------------------------------
@dataclass
class CodecConfig:
    num_quantizers: int = 8
    codebook_size: int = 1024
    codebook_dim: int = 512
    code_dim: int = 3072
    d_model: int = 768
    heads: int = 12
    ffn_dim: int = 3072
    post_rvq_layers: int = 4
    acoustic_layers: int = 12
    mel_bins: int = 80
    n_fft: int = 960
    hop: int = 240
    vocos_dim: int = 512
    vocos_intermediate: int = 4096
    vocos_layers: int = 30

    @property
    def samples_per_frame(self) -> int:
        return 4 * 2 * self.hop


def resolve_weight_norm(raw: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    out = {}
    for k, v in raw.items():
        if k.endswith(".weight_g"):
            base = k[:-len(".weight_g")]
            if base + ".weight_v" not in raw:
                raise LoadError(f"codec: {base}.weight_g without weight_v")
            wv = raw[base + ".weight_v"].float()
            norm = wv.flatten(1).norm(dim=1).view(-1, *([1] * (wv.dim() - 1)))
            out[base + ".weight"] = wv * (v.float() / norm)
        elif not k.endswith(".weight_v"):
            out[k] = v.float() if v.is_floating_point() else v
    return out


def sinusoids(length: int, channels: int) -> torch.Tensor:
    half = channels // 2
    inv = torch.exp(-(math.log(10000.0) / (half - 1)) * torch.arange(half, dtype=torch.float64))
    ang = torch.arange(length, dtype=torch.float64)[:, None] * inv[None]
    return torch.cat([ang.sin(), ang.cos()], 1).float()


def hann_window(n: int) -> torch.Tensor:
    return (0.5 - 0.5 * torch.cos(2.0 * math.pi * torch.arange(n, dtype=torch.float64) / n)).float()


def idft_basis(n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Real inverse DFT as two [n, n / 2 + 1] matrices: x = cos @ re - sin @ im."""
    k = torch.arange(n // 2 + 1, dtype=torch.float64)
    a = torch.where((k == 0) | (k == n // 2), 1.0, 2.0)
    th = 2.0 * math.pi * torch.arange(n, dtype=torch.float64)[:, None] * k[None] / n
    return (a * th.cos() / n).float(), (a * th.sin() / n).float()


def overlap_add(frames: torch.Tensor, window: torch.Tensor, hop: int) -> torch.Tensor:
    """[T, n] windowed overlap-add, divided by the summed squared window, (n - hop) / 2 samples trimmed at both ends."""
    T, n = frames.shape
    if T == 0:
        return frames.new_zeros(0)
    out_len = (T - 1) * hop + n
    y = F.fold((frames * window).t()[None], (1, out_len), (1, n), stride=(1, hop)).reshape(-1)
    env = F.fold((window * window)[:, None].expand(n, T)[None], (1, out_len), (1, n), stride=(1, hop)).reshape(-1)
    pad = (n - hop) // 2
    y, env = y[pad:out_len - pad], env[pad:out_len - pad]
    return torch.where(env > 1e-11, y / env.clamp(min=1e-11), torch.zeros_like(y))


class XyTokenizerCodec:
    def __init__(self, weights: dict[str, torch.Tensor], cfg: CodecConfig | None = None, device="cpu"):
        self.cfg, self.device = cfg or CodecConfig(), torch.device(device)
        keep = ("quantizer.", "post_rvq_adapter.", "upsample.", "acoustic_decoder.", "enhanced_vocos.")
        raw = {k: v for k, v in weights.items() if k.startswith(keep) and not k.endswith((".inited", ".cluster_size", ".embed_avg"))}
        self.w = {k: v.to(self.device) for k, v in resolve_weight_norm(raw).items()}
        self.cos, self.sin = (t.to(self.device) for t in idft_basis(self.cfg.n_fft))
        self.window = hann_window(self.cfg.n_fft).to(self.device)

    def _lin(self, x, p, bias=True):
        return F.linear(x, self.w[p + ".weight"], self.w.get(p + ".bias") if bias else None)

    def _ln(self, x, p, eps=1e-5):
        return F.layer_norm(x, (x.shape[-1],), self.w[p + ".weight"], self.w[p + ".bias"], eps)

    def _layer(self, x, p):
        H = self.cfg.heads
        h = self._ln(x, p + ".self_attn_layer_norm")
        B, T, D = h.shape
        hs = lambda t: t.view(B, T, H, D // H).transpose(1, 2)                          # noqa: E731
        q, k, v = hs(self._lin(h, p + ".self_attn.q_proj")), hs(self._lin(h, p + ".self_attn.k_proj", False)), hs(self._lin(h, p + ".self_attn.v_proj"))
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, D)
        x = x + self._lin(a, p + ".self_attn.out_proj")
        return x + self._lin(F.gelu(self._lin(self._ln(x, p + ".final_layer_norm"), p + ".fc1")), p + ".fc2")

    def _stack(self, x, p, layers):
        x = x + sinusoids(x.shape[1], x.shape[2]).to(x.device)[None]
        for i in range(layers):
            x = self._layer(x, f"{p}.layers.{i}")
        return self._ln(x, p + ".layer_norm")

    @torch.no_grad()
    def mel(self, frames: list[list[int]]) -> torch.Tensor:
        c, w = self.cfg, self.w
        codes = torch.tensor(frames, dtype=torch.int64, device=self.device).clamp(max=c.codebook_size - 1)       # [T, nq]
        z = sum(w[f"quantizer.quantizers.{q}.codebook"][codes[:, q]] for q in range(min(c.num_quantizers, codes.shape[1])))
        x = F.conv1d(z.t()[None], w["quantizer.output_proj.weight"], w["quantizer.output_proj.bias"])            # [1, 3072, T]
        h = self._lin(x.transpose(1, 2), "post_rvq_adapter.proj")
        h = self._lin(self._stack(h, "post_rvq_adapter", c.post_rvq_layers), "post_rvq_adapter.out_proj").transpose(1, 2)
        h = F.conv_transpose1d(h, w["upsample.up_conv.weight"], None, stride=4)                                    # [1, 768, 4T]
        L = h.shape[2]
        h = self._stack(h.transpose(1, 2), "acoustic_decoder", c.acoustic_layers).transpose(1, 2)
        h = F.gelu(F.conv_transpose1d(h, w["acoustic_decoder.deconv1.weight"], w["acoustic_decoder.deconv1.bias"], stride=2))
        h = F.gelu(F.conv_transpose1d(h, w["acoustic_decoder.deconv2.weight"], w["acoustic_decoder.deconv2.bias"], stride=1))
        return h[:, :, :2 * L]

    @torch.no_grad()
    def vocode(self, mel: torch.Tensor) -> torch.Tensor:
        c, w, b = self.cfg, self.w, "enhanced_vocos.backbone."
        x = F.conv1d(mel, w[b + "embed.weight"], w[b + "embed.bias"], padding=3)
        x = self._ln(x.transpose(1, 2), b + "norm", 1e-6).transpose(1, 2)
        for i in range(c.vocos_layers):
            p = f"{b}convnext.{i}"
            h = F.conv1d(x, w[p + ".dwconv.weight"], w[p + ".dwconv.bias"], padding=3, groups=x.shape[1]).transpose(1, 2)
            h = self._lin(F.gelu(self._lin(self._ln(h, p + ".norm", 1e-6), p + ".pwconv1")), p + ".pwconv2") * w[p + ".gamma"]
            x = x + h.transpose(1, 2)
        coeffs = self._lin(self._ln(x.transpose(1, 2), b + "final_layer_norm", 1e-6), "enhanced_vocos.head.out")[0]
        nb = c.n_fft // 2 + 1
        mag, phase = coeffs[:, :nb].exp().clamp(max=1e2), coeffs[:, nb:]
        frames = (mag * phase.cos()) @ self.cos.t() - (mag * phase.sin()) @ self.sin.t()                          # [T, n_fft]
        return overlap_add(frames, self.window, c.hop)

    def decode_frames(self, frames: list[list[int]], cancel=lambda: False) -> torch.Tensor | None:
        if not frames:
            return torch.zeros(0)
        if cancel():
            return None
        mel = self.mel(frames)
        if cancel():
            return None
        return self.vocode(mel).float().cpu()


def load_codec_weights(path: Path) -> tuple[dict[str, torch.Tensor], CodecConfig]:
    path = Path(path)
    if path.suffix == ".safetensors":
        from ..io.safetensors_io import load_file

        w = load_file(path)
        cfg = CodecConfig()
        if "swb_codec_config" in w:
            cfg = CodecConfig(*[int(v) for v in w.pop("swb_codec_config").tolist()])
        return w, cfg
    if not path.is_file():
        raise LoadError(f"{MODEL_ID}: codec checkpoint {path} not found")
    sd = torch.load(path, map_location="cpu", weights_only=True)
    return sd.get("generator", sd), CodecConfig()


# ---- generator ------------------------------------------------------------------------------------------------------------
def script_to_dialogue(script: list[dict]) -> str:
    speakers, out = [], []
    for i, seg in enumerate(script):
        name = seg.get("speaker")
        if name is not None:
            if name not in speakers:
                speakers.append(name)
            tag = speakers.index(name)
        else:
            tag = i
        out.append(f"[S{tag % MAX_SPEAKERS + 1}]{str(seg.get('text', '')).strip()}")
    return "".join(out)


def request_text(req: GenerationRequest) -> str:
    a = req.audio
    return script_to_dialogue(a.script) if a is not None and a.script else req.prompt


def position_budget(req: GenerationRequest, channels: int) -> int:
    a = req.audio
    secs = a.target_duration if a is not None and a.target_duration is not None else DEFAULT_SECONDS
    return max(int(math.ceil(secs * FRAME_RATE_HZ)), 64) + channels


def moss_ttsd_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family=FAMILY, backend=backend, modality=Modality.AUDIO,
        capabilities=Capabilities(
            supports_negative_prompt=False, supports_guidance=False, supports_true_cfg=False, conditioning=[],
            supports_lora=False, supports_lokr=False, samplers=[], schedulers=[], supported_guidance_methods=[],
            min_size=0, max_size=0, max_count=1, audio_sample_rates=[SAMPLE_RATE], max_audio_duration_secs=MAX_DURATION_SECS,
            audio_voices=[], audio_languages=list(LANGUAGES), supports_multi_speaker=True, max_speakers=MAX_SPEAKERS),
        required_components=[CODEC_COMPONENT_ID])


class MossTtsdGenerator(Generator):
    def __init__(self, root: Path, codec_path: Path, backend: str, prefix: str = ""):
        self.root, self.codec_path, self.backend = Path(root), Path(codec_path), backend
        self._descriptor = moss_ttsd_descriptor(backend, prefix)
        self._loaded, self._codec = None, None

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        a = req.audio
        if not req.prompt.strip() and not (a is not None and a.script):
            raise InferenceError(f"{mid}: prompt or a multi-speaker audio.script (the text to speak) must not be empty")
        self._descriptor.capabilities.validate_request_audio(mid, req)

    def _device(self) -> str:
        return "cuda" if self.backend == "b200" else "cpu"

    def pipeline(self):
        if self._loaded is None:
            import tokenizers

            from ..io.safetensors_io import load_file

            cj, tk, wf = self.root / "config.json", self.root / "tokenizer.json", self.root / MODEL_WEIGHTS
            for f in (cj, tk, wf):
                if not f.is_file():
                    raise LoadError(f"{MODEL_ID}: {f} missing (the snapshot must supply config.json, tokenizer.json and {MODEL_WEIGHTS})")
            cfg = MossTtsdConfig.from_json(json.loads(cj.read_text(encoding="utf-8")))
            self._loaded = (Backbone(cfg, load_file(wf), self._device()), tokenizers.Tokenizer.from_file(str(tk)))
        return self._loaded

    def codec(self) -> XyTokenizerCodec:
        if self._codec is None:
            w, cfg = load_codec_weights(self.codec_path)
            self._codec = XyTokenizerCodec(w, cfg, self._device())
        return self._codec

    def rvq_frames(self, req: GenerationRequest, on_progress=lambda p: None) -> tuple[list[list[int]], str]:
        self.validate(req)
        if req.cancel.is_cancelled():
            raise Canceled(f"{MODEL_ID}: cancelled")
        backbone, tok = self.pipeline()
        grid = build_prompt_grid(tok, backbone.cfg, request_text(req))
        budget = position_budget(req, backbone.cfg.channels)
        res = run_decoder(backbone, grid, budget, req.seed if req.seed is not None else DEFAULT_SAMPLING_SEED,
                          req.cancel.is_cancelled, lambda step: on_progress(ProgressStep(step + 1, budget)))
        if res is None:
            raise Canceled(f"{MODEL_ID}: cancelled")
        return res

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        frames, _ = self.rvq_frames(req, on_progress)
        codec = self.codec()
        on_progress(ProgressDecoding())
        wav = codec.decode_frames(frames, req.cancel.is_cancelled)
        if wav is None:
            raise Canceled(f"{MODEL_ID}: cancelled while decoding")
        return GenerationOutput(audio=AudioTrack(SAMPLE_RATE, 1, wav.tolist()))


def registration(backend: str) -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> MossTtsdGenerator:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise LoadError(f"{mid} expects a snapshot directory (config.json + {MODEL_WEIGHTS} + tokenizer.json), not a single file")
        if spec.quantize is not None:
            raise Unsupported(f"{mid} does not support on-the-fly quantization")
        if spec.adapters:
            raise Unsupported(f"{mid} does not support LoRA/LoKr adapters")
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid} does not support control/IP-adapter overlays")
        reject_unknown_components(spec.components, [CODEC_COMPONENT_ID], mid)
        src = require_component(spec.components, CODEC_COMPONENT_ID, mid)
        codec = Path(src.path) if src.is_file else Path(src.path) / CODEC_CHECKPOINT_FILE
        if not src.is_file and not codec.is_file() and (Path(src.path) / "xy_tokenizer.safetensors").is_file():
            codec = Path(src.path) / "xy_tokenizer.safetensors"
        return MossTtsdGenerator(Path(spec.weights.path), codec, backend, prefix)

    return Registration(descriptor=lambda: moss_ttsd_descriptor(backend, prefix), load=load)


# ---- synthetic checkpoints ------------------------------------------------------------------------------------------------
def random_codec_weights(cfg: CodecConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)                      # noqa: E731
    w: dict[str, torch.Tensor] = {}

    def lin(p, o, i, bias=True):
        w[p + ".weight"] = rn(o, i) / math.sqrt(i)
        if bias:
            w[p + ".bias"] = rn(o) * 0.02

    def ln(p, d):
        w[p + ".weight"], w[p + ".bias"] = 1 + rn(d) * 0.05, rn(d) * 0.02

    def layer(p):
        ln(p + ".self_attn_layer_norm", cfg.d_model)
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            lin(f"{p}.self_attn.{n}", cfg.d_model, cfg.d_model, bias=n != "k_proj")
        ln(p + ".final_layer_norm", cfg.d_model)
        lin(p + ".fc1", cfg.ffn_dim, cfg.d_model)
        lin(p + ".fc2", cfg.d_model, cfg.ffn_dim)

    for q in range(cfg.num_quantizers):
        w[f"quantizer.quantizers.{q}.codebook"] = rn(cfg.codebook_size, cfg.codebook_dim)
    v = rn(cfg.code_dim, cfg.codebook_dim, 1) / math.sqrt(cfg.codebook_dim)
    w["quantizer.output_proj.weight_v"], w["quantizer.output_proj.weight_g"] = v, v.flatten(1).norm(dim=1).view(-1, 1, 1) * 1.1
    w["quantizer.output_proj.bias"] = rn(cfg.code_dim) * 0.02
    lin("post_rvq_adapter.proj", cfg.d_model, cfg.code_dim)
    lin("post_rvq_adapter.out_proj", cfg.code_dim, cfg.d_model)
    ln("post_rvq_adapter.layer_norm", cfg.d_model)
    for i in range(cfg.post_rvq_layers):
        layer(f"post_rvq_adapter.layers.{i}")
    w["upsample.up_conv.weight"] = rn(cfg.code_dim, cfg.d_model, 4) / math.sqrt(cfg.code_dim)
    ln("acoustic_decoder.layer_norm", cfg.d_model)
    for i in range(cfg.acoustic_layers):
        layer(f"acoustic_decoder.layers.{i}")
    w["acoustic_decoder.deconv1.weight"], w["acoustic_decoder.deconv1.bias"] = rn(cfg.d_model, cfg.d_model, 3) / math.sqrt(cfg.d_model * 3), rn(cfg.d_model) * 0.02
    w["acoustic_decoder.deconv2.weight"], w["acoustic_decoder.deconv2.bias"] = rn(cfg.d_model, cfg.mel_bins, 3) / math.sqrt(cfg.d_model * 3), rn(cfg.mel_bins) * 0.02
    b = "enhanced_vocos.backbone."
    w[b + "embed.weight"], w[b + "embed.bias"] = rn(cfg.vocos_dim, cfg.mel_bins, 7) / math.sqrt(cfg.mel_bins * 7), rn(cfg.vocos_dim) * 0.02
    ln(b + "norm", cfg.vocos_dim)
    ln(b + "final_layer_norm", cfg.vocos_dim)
    for i in range(cfg.vocos_layers):
        p = f"{b}convnext.{i}"
        w[p + ".dwconv.weight"], w[p + ".dwconv.bias"] = rn(cfg.vocos_dim, 1, 7) / math.sqrt(7), rn(cfg.vocos_dim) * 0.02
        ln(p + ".norm", cfg.vocos_dim)
        lin(p + ".pwconv1", cfg.vocos_intermediate, cfg.vocos_dim)
        lin(p + ".pwconv2", cfg.vocos_dim, cfg.vocos_intermediate)
        w[p + ".gamma"] = torch.full((cfg.vocos_dim,), 0.1)
    lin("enhanced_vocos.head.out", cfg.n_fft + 2, cfg.vocos_dim)
    w["enhanced_vocos.head.out.weight"] *= 0.1
    return w


def write_synthetic_snapshot(root, seed: int = 0) -> tuple[Path, Path]:
    """(model snapshot, codec file): a 2-layer backbone with a toy byte-level tokenizer that knows the markup tokens, 4
    channels, and a small codec with the real resampling factors."""
    import tokenizers
    from tokenizers import decoders, models, pre_tokenizers, trainers

    from ..io.safetensors_io import save_file
    from ..models.config import ModelConfig
    from ..models.oracle import random_llama_weights

    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    specials = ["<|begin_of_style|>", "<|end_of_style|>", "<|begin_of_text|>", "<|end_of_text|>", "<|begin_of_speech|>", "<speaker1>",
                "<speaker2>"]
    tok = tokenizers.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(["hello there how are you", "fine thanks and you", DEFAULT_SYSTEM_PROMPT],
                            trainers.BpeTrainer(vocab_size=330, special_tokens=specials, initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tok.save(str(root / "tokenizer.json"))
    text_vocab = tok.get_vocab_size()
    codes = 16
    cfg = dict(model_type="moss_ttsd", vocab_size=text_vocab + codes + 8, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=2, num_key_value_heads=1, head_dim=16, channels=4, speech_vocab_size=codes + 1, speech_pad_token=codes,
               speech_token_range=[text_vocab, text_vocab + codes], speech_eos_token=text_vocab + codes + 2, bos_token_id=text_vocab + codes + 3)
    (root / "config.json").write_text(json.dumps(cfg))
    lcfg = ModelConfig.from_json({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", **{k: cfg[k] for k in (
        "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim")},
        "rms_norm_eps": 1e-6, "rope_theta": 1e6, "tie_word_embeddings": True, "max_position_embeddings": 4096})
    lw = random_llama_weights(lcfg, seed, std=0.3)
    w = {"model.language_model." + k[len("model."):]: v for k, v in lw.items() if k.startswith("model.") and "embed_tokens" not in k}
    g = torch.Generator().manual_seed(seed + 1)
    w["model.embedding_list.0.weight"] = lw["model.embed_tokens.weight"]
    for c in range(1, cfg["channels"]):
        w[f"model.embedding_list.{c}.weight"] = torch.randn(codes + 1, 32, generator=g) * 0.3
    save_file(w, root / MODEL_WEIGHTS)
    ccfg = CodecConfig(num_quantizers=4, codebook_size=codes, codebook_dim=8, code_dim=24, d_model=16, heads=2, ffn_dim=32, post_rvq_layers=1,
                       acoustic_layers=1, mel_bins=6, n_fft=960, hop=240, vocos_dim=8, vocos_intermediate=16, vocos_layers=2)
    cw = random_codec_weights(ccfg, seed + 2)
    cw["swb_codec_config"] = torch.tensor([getattr(ccfg, f) for f in CodecConfig.__dataclass_fields__])
    codec = root.parent / (root.name + "_codec.safetensors")
    save_file(cw, codec)
    return root, codec
