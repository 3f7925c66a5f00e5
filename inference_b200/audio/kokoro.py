"""Kokoro-82M text-to-speech generator `kokoro_82m` (parity: candle-audio-kokoro/src/{albert,text_encoder,predictor,
decoder,nn,pipeline,model,weights,g2p}.rs).

A StyleTTS2-derived stack, all of it here: phonemes -> PL-BERT (ALBERT: one shared layer run N times) -> prosody
predictor (style-conditioned BiLSTM / AdaLayerNorm duration encoder, per-token durations, F0 and energy curves through
AdaIN residual stacks) -> text encoder (conv + channel LayerNorm + BiLSTM) expanded by the durations -> styled decoder ->
iSTFT-Net vocoder (nine-harmonic sine source from the F0 curve + seeded noise, its 20-point STFT as a side input at
every upsampling stage, AdaIN Snake residual blocks, magnitude / phase head, inverse STFT). 24 kHz mono, 600 samples
per prosody frame. Voices are style packs [510, 1, 256] indexed by token count: first 128 numbers style the decoder,
the last 128 the prosody predictor.

Checkpoint: `kokoro-v1_0.pth` (five sections `bert`, `bert_encoder`, `predictor`, `text_encoder`, `decoder`; old-style
weight norm `weight_g` / `weight_v` folded at load) or `kokoro.safetensors` with `<section>.<key>` names; `config.json`
(dimensions + the phoneme vocabulary); `voices/<name>.pt` or `.safetensors`. Phonemisation: a lexicon
`g2p/<us|gb>.json` (word -> phoneme string) when the snapshot has one, letter-to-sound fallback otherwise; characters of
the input that already are vocabulary symbols (an IPA script) pass through unchanged.

The network is small (82 M parameters, batch 1): recurrent layers and 1-D convolutions run through the framework's
calls on either backend in fp32; the harmonic source and the tiny STFT pair are vectorised tensor code."""
from __future__ import annotations

import json
import math
import re
from dataclasses import dataclass, field
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

MODEL_ID, SAMPLE_RATE, SAMPLES_PER_FRAME, STAGES = "kokoro_82m", 24_000, 600, 5
CHECKPOINT_FILE, MAX_DURATION_SECS, DEFAULT_VOICE = "kokoro-v1_0.pth", 30.0, "af_heart"
VOICES = ["af_alloy", "af_aoede", "af_bella", "af_heart", "af_jessica", "af_kore", "af_nicole", "af_nova", "af_river",
          "af_sarah", "af_sky", "am_adam", "am_echo", "am_eric", "am_fenrir", "am_liam", "am_michael", "am_onyx", "am_puck",
          "am_santa", "bf_alice", "bf_emma", "bf_isabella", "bf_lily", "bm_daniel", "bm_fable", "bm_george", "bm_lewis"]
LANGUAGES = ["en", "en-us", "en-gb"]
KOKORO_LICENSE = WeightLicense("Apache-2.0", "Apache License 2.0", "https://huggingface.co/hexgrad/Kokoro-82M",
                               "Kokoro-82M (c) hexgrad - licensed under Apache-2.0", True)
SINE_AMP, NOISE_STD, VOICED_THRESHOLD, HARMONICS = 0.1, 0.003, 10.0, 9


@dataclass
class KokoroConfig:
    hidden_dim: int = 512
    style_dim: int = 128
    max_dur: int = 50
    n_layer: int = 3
    n_token: int = 178
    text_encoder_kernel_size: int = 5
    plbert: dict = field(default_factory=lambda: dict(hidden_size=768, num_attention_heads=12, intermediate_size=2048,
                                                      max_position_embeddings=512, num_hidden_layers=12))
    istftnet: dict = field(default_factory=lambda: dict(
        upsample_kernel_sizes=[20, 12], upsample_rates=[10, 6], gen_istft_hop_size=5, gen_istft_n_fft=20,
        resblock_dilation_sizes=[[1, 3, 5], [1, 3, 5], [1, 3, 5]], resblock_kernel_sizes=[3, 7, 11], upsample_initial_channel=512))
    vocab: dict = field(default_factory=dict)
    decoder_width: int = 1024            # fixed in the published model; smaller in synthetic snapshots

    @staticmethod
    def from_json(j: dict) -> "KokoroConfig":
        for k in ("istftnet", "plbert", "vocab"):
            if k not in j:
                raise LoadError(f"kokoro config.json: missing {k} block")
        return KokoroConfig(**{k: j[k] for k in KokoroConfig.__dataclass_fields__ if k in j})

    def phonemes_to_ids(self, phonemes: str) -> list[int]:
        return [self.vocab[c] for c in phonemes if c in self.vocab]


# ---- building blocks ----------------------------------------------------------------------------------------------------
class _W:
    def __init__(self, weights: dict[str, torch.Tensor], device):
        self.device = torch.device(device)
        w = {}
        for k, v in weights.items():                      # old-style weight norm: w = g * v / ||v|| per output channel
            if k.endswith(".weight_g"):
                base = k[: -len("_g")]
                vv = weights[base + "_v"].float()
                norm = vv.reshape(vv.shape[0], -1).norm(dim=1).reshape(-1, *([1] * (vv.dim() - 1)))
                w[base] = v.float() * vv / norm
            elif not k.endswith(".weight_v"):
                w[k] = v.float() if v.is_floating_point() else v
        self.w = {k: v.to(self.device).contiguous() for k, v in w.items()}

    def lin(self, x, p):
        return F.linear(x, self.w[p + ".weight"], self.w.get(p + ".bias"))

    def conv(self, x, p, **kw):
        return F.conv1d(x, self.w[p + ".weight"], self.w.get(p + ".bias"), **kw)

    def bilstm(self, x, p):
        """x [1, T, in] -> [1, T, 2 * hidden] (torch.nn.LSTM parameter names, bidirectional, one layer)."""
        ws = [self.w[f"{p}.{n}{sfx}"] for sfx in ("", "_reverse") for n in ("weight_ih_l0", "weight_hh_l0", "bias_ih_l0", "bias_hh_l0")]
        hid = ws[1].shape[1]
        h0 = torch.zeros(2, x.shape[0], hid, device=x.device)
        out, _, _ = torch._VF.lstm(x, (h0, h0.clone()), ws, True, 1, 0.0, False, True, True)
        return out

    def adain(self, x, s, p):                               # x [1, C, T], s [1, style]
        h = self.lin(s, p + ".fc")
        c = h.shape[1] // 2
        xn = (x - x.mean(2, keepdim=True)) / torch.sqrt(x.var(2, unbiased=False, keepdim=True) + 1e-5)
        return xn * (1 + h[:, :c, None]) + h[:, c:, None]

    def ada_layer_norm(self, x, s, p):                      # x [1, C, T]: normalise over channels
        h = self.lin(s, p + ".fc")
        c = h.shape[1] // 2
        xt = F.layer_norm(x.transpose(1, 2), (x.shape[1],), eps=1e-5)
        return (xt * (1 + h[:, None, :c]) + h[:, None, c:]).transpose(1, 2)

    def adain_resblk(self, x, s, p):
        """AdainResBlk1d: [AdaIN, LeakyReLU 0.2, (depthwise stride-2 transposed conv), conv3] x 2 + shortcut, / sqrt 2."""
        up = p + ".pool.weight" in self.w
        h = F.leaky_relu(self.adain(x, s, p + ".norm1"), 0.2)
        if up:
            h = F.conv_transpose1d(h, self.w[p + ".pool.weight"], self.w.get(p + ".pool.bias"), stride=2, padding=1,
                                   output_padding=1, groups=h.shape[1])
        h = self.conv(h, p + ".conv1", padding=1)
        h = self.conv(F.leaky_relu(self.adain(h, s, p + ".norm2"), 0.2), p + ".conv2", padding=1)
        sc = F.interpolate(x, scale_factor=2.0, mode="nearest") if up else x
        if p + ".conv1x1.weight" in self.w:
            sc = self.conv(sc, p + ".conv1x1")
        return (h + sc) / math.sqrt(2.0)

    def snake_resblock(self, x, s, p, kernel: int, dilations):
        for i, d in enumerate(dilations):
            a1, a2 = self.w[f"{p}.alpha1.{i}"], self.w[f"{p}.alpha2.{i}"]
            t = self.adain(x, s, f"{p}.adain1.{i}")
            t = t + torch.sin(t * a1) ** 2 / a1
            t = self.conv(t, f"{p}.convs1.{i}", padding=(kernel * d - d) // 2, dilation=d)
            t = self.adain(t, s, f"{p}.adain2.{i}")
            t = t + torch.sin(t * a2) ** 2 / a2
            x = x + self.conv(t, f"{p}.convs2.{i}", padding=(kernel - 1) // 2)
        return x


def gelu_new(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def stft_small(x: torch.Tensor, n_fft: int, hop: int):
    """Centred (reflect-padded), periodic-Hann STFT of a 1-D signal -> (magnitude, phase) [bins, frames]."""
    win = torch.hann_window(n_fft, periodic=True, device=x.device)
    spec = torch.stft(x, n_fft, hop, n_fft, win, center=True, pad_mode="reflect", return_complex=True)
    return spec.abs(), torch.angle(spec)


def istft_small(mag: torch.Tensor, phase: torch.Tensor, n_fft: int, hop: int) -> torch.Tensor:
    win = torch.hann_window(n_fft, periodic=True, device=mag.device)
    return torch.istft(torch.polar(mag, phase), n_fft, hop, n_fft, win, center=True)


def harmonic_source(f0: torch.Tensor, scale: int, l_weight: torch.Tensor, l_bias: float, gen: torch.Generator) -> torch.Tensor:
    """Frame-rate F0 [F] -> excitation [F * scale]: nine harmonics whose phase is the running sum of f0 * k / 24000
    (mod 1) per frame, linearly interpolated to the sample rate (half-pixel centres) and multiplied by `scale`; voiced
    samples are sines of amplitude 0.1 plus noise of deviation 0.003, unvoiced ones noise of deviation 0.1 / 3; a learned
    9 -> 1 mix and tanh close it."""
    Fn = f0.shape[0]
    k = torch.arange(1, HARMONICS + 1, dtype=torch.float64)
    rad = torch.remainder(f0.double()[None, :] * k[:, None] / SAMPLE_RATE, 1.0)
    phase = torch.cumsum(rad, dim=1) * 2.0 * math.pi                                    # [9, F]
    c = ((torch.arange(Fn * scale, dtype=torch.float64) + 0.5) / scale - 0.5).clamp(0.0, Fn - 1.0)
    i0 = c.floor().long().clamp(max=max(Fn - 2, 0))
    frac = c - i0
    i1 = (i0 + 1).clamp(max=Fn - 1)
    ph = phase[:, i0] * (1.0 - frac) + phase[:, i1] * frac
    sines = torch.sin(ph * scale).float() * SINE_AMP                                    # [9, n]
    uv = (f0 > VOICED_THRESHOLD).float().repeat_interleave(scale)[None]
    noise = torch.randn(HARMONICS, Fn * scale, generator=gen) * (uv * NOISE_STD + (1.0 - uv) * SINE_AMP / 3.0)
    return torch.tanh((l_weight.reshape(-1, 1).cpu() * (sines * uv + noise)).sum(0) + l_bias)


class KokoroPipeline:
    def __init__(self, cfg: KokoroConfig, sections: dict[str, dict[str, torch.Tensor]], device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        strip = lambda d: {(k[len("module."):] if k.startswith("module.") else k): v for k, v in d.items()}      # noqa: E731
        self.bert, self.bert_encoder = _W(strip(sections["bert"]), device), _W(strip(sections["bert_encoder"]), device)
        self.pred, self.text, self.dec = (_W(strip(sections[k]), device) for k in ("predictor", "text_encoder", "decoder"))

    # ---- stages ---------------------------------------------------------------------------------------------------
    def _plbert(self, ids: torch.Tensor) -> torch.Tensor:
        b, pc = self.bert, self.cfg.plbert
        T = ids.shape[1]
        e = (b.w["embeddings.word_embeddings.weight"][ids] + b.w["embeddings.position_embeddings.weight"][:T][None]
             + b.w["embeddings.token_type_embeddings.weight"][0][None, None])
        e = F.layer_norm(e, (e.shape[-1],), b.w["embeddings.LayerNorm.weight"], b.w["embeddings.LayerNorm.bias"], 1e-12)
        h = b.lin(e, "encoder.embedding_hidden_mapping_in")
        L, nh = "encoder.albert_layer_groups.0.albert_layers.0", pc["num_attention_heads"]
        for _ in range(pc["num_hidden_layers"]):
            q, k, v = (b.lin(h, f"{L}.attention.{n}").reshape(1, T, nh, -1).transpose(1, 2) for n in ("query", "key", "value"))
            ctx = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(1, T, -1)
            a = b.lin(ctx, L + ".attention.dense") + h
            a = F.layer_norm(a, (a.shape[-1],), b.w[L + ".attention.LayerNorm.weight"], b.w[L + ".attention.LayerNorm.bias"], 1e-12)
            f = b.lin(gelu_new(b.lin(a, L + ".ffn")), L + ".ffn_output") + a
            h = F.layer_norm(f, (f.shape[-1],), b.w[L + ".full_layer_layer_norm.weight"], b.w[L + ".full_layer_layer_norm.bias"], 1e-12)
        return h

    def _duration_encoder(self, d_en: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
        p, T = self.pred, d_en.shape[2]
        st = s[:, :, None].expand(-1, -1, T)
        x = torch.cat([d_en, st], 1)
        for layer in range(self.cfg.n_layer):
            out = p.bilstm(x.transpose(1, 2), f"text_encoder.lstms.{2 * layer}").transpose(1, 2)
            x = torch.cat([p.ada_layer_norm(out, s, f"text_encoder.lstms.{2 * layer + 1}"), st], 1)
        return x.transpose(1, 2)                                                          # [1, T, d + style]

    def raw_durations(self, tokens: list[int], ref_s: torch.Tensor) -> torch.Tensor:
        return self._durations(self._ids(tokens), ref_s[:, self.cfg.style_dim:].to(self.device))[1]

    def _ids(self, tokens):
        return torch.tensor([[0, *tokens, 0]], dtype=torch.int64, device=self.device)

    def _durations(self, ids, s_pros):
        d_en = F.linear(self._plbert(ids), self.bert_encoder.w["weight"], self.bert_encoder.w["bias"]).transpose(1, 2)
        d = self._duration_encoder(d_en, s_pros)
        x = self.pred.bilstm(d, "lstm")
        return d, torch.sigmoid(self.pred.lin(x, "duration_proj.linear_layer")).sum(2)[0]

    def natural_duration_secs(self, raw: torch.Tensor) -> float:
        return float(torch.round(raw).clamp(min=1.0).sum()) * SAMPLES_PER_FRAME / SAMPLE_RATE

    @torch.no_grad()
    def synthesize(self, tokens: list[int], ref_s: torch.Tensor, speed: float, seed: int, stage=lambda i: None) -> torch.Tensor:
        cfg = self.cfg
        if not tokens:
            raise InferenceError("kokoro: no phonemes survived tokenization (unsupported script?)")
        if len(tokens) + 2 > cfg.plbert["max_position_embeddings"]:
            raise InferenceError(f"kokoro: {len(tokens) + 2} phoneme tokens exceed the model context of "
                                 f"{cfg.plbert['max_position_embeddings']} (split the script)")
        if not (math.isfinite(speed) and 0.1 <= speed <= 10.0):
            raise InferenceError(f"kokoro: speed {speed} out of range")
        gen = torch.Generator().manual_seed(seed & 0x7FFFFFFFFFFFFFFF)
        ref_s = ref_s.to(self.device).float().reshape(1, -1)
        s_dec, s_pros = ref_s[:, : cfg.style_dim], ref_s[:, cfg.style_dim:]
        ids = self._ids(tokens)
        d, raw = self._durations(ids, s_pros)
        stage(1)
        dur = torch.round(raw / speed).clamp(min=1.0).long()                              # round-half-even like the reference
        frame_token = torch.repeat_interleave(torch.arange(len(dur), device=self.device), dur)
        stage(2)
        en = d[0][frame_token].t()[None]                                                  # [1, d + style, F]
        p = self.pred
        x = p.bilstm(en.transpose(1, 2), "shared").transpose(1, 2)
        f0, n = x, x
        for i in range(3):
            f0, n = p.adain_resblk(f0, s_pros, f"F0.{i}"), p.adain_resblk(n, s_pros, f"N.{i}")
        f0, n = p.conv(f0, "F0_proj")[0, 0], p.conv(n, "N_proj")[0, 0]                    # [2F] each
        stage(3)
        t = self.text
        h = t.w["embedding.weight"][ids].transpose(1, 2)
        for i in range(cfg.n_layer):
            h = t.conv(h, f"cnn.{i}.0", padding=(cfg.text_encoder_kernel_size - 1) // 2)
            hn = F.layer_norm(h.transpose(1, 2), (h.shape[1],), t.w[f"cnn.{i}.1.gamma"], t.w[f"cnn.{i}.1.beta"], 1e-5)
            h = F.leaky_relu(hn.transpose(1, 2), 0.2)
        t_en = t.bilstm(h.transpose(1, 2), "lstm")[0]                                     # [T, C]
        asr = t_en[frame_token].t()[None]                                                 # [1, C, F]
        stage(4)
        samples = self._decode(asr, f0, n, s_dec, gen)
        want = int(dur.sum()) * SAMPLES_PER_FRAME
        if samples.numel() != want:
            raise InferenceError(f"kokoro: vocoder produced {samples.numel()} samples for {int(dur.sum())} frames (expected {want})")
        if not torch.isfinite(samples).all():
            raise InferenceError("kokoro: non-finite samples")
        stage(5)
        return samples

    def _decode(self, asr, f0, n, s, gen):
        d, ic = self.dec, self.cfg.istftnet
        f0d = d.conv(f0[None, None], "F0_conv", stride=2, padding=1)
        nd = d.conv(n[None, None], "N_conv", stride=2, padding=1)
        x = d.adain_resblk(torch.cat([asr, f0d, nd], 1), s, "encode")
        res = d.conv(asr, "asr_res.0")
        for i in range(4):
            x = d.adain_resblk(torch.cat([x, res, f0d, nd], 1), s, f"decode.{i}")
        # ---- generator ----
        g = "generator."
        rates, ksz = ic["upsample_rates"], ic["upsample_kernel_sizes"]
        n_fft, hop = ic["gen_istft_n_fft"], ic["gen_istft_hop_size"]
        scale = math.prod(rates) * hop
        har = harmonic_source(f0.cpu(), scale, d.w[g + "m_source.l_linear.weight"], float(d.w[g + "m_source.l_linear.bias"]), gen)
        mag, ph = stft_small(har.to(self.device), n_fft, hop)
        har_spec = torch.cat([mag, ph], 0)[None]                                          # [1, n_fft + 2, frames]
        nk, n_up = len(ic["resblock_kernel_sizes"]), len(rates)
        for i in range(n_up):
            x = F.leaky_relu(x, 0.1)
            if i + 1 < n_up:
                sf = math.prod(rates[i + 1:])
                xs = d.conv(har_spec, f"{g}noise_convs.{i}", stride=sf, padding=(sf + 1) // 2)
                xs = d.snake_resblock(xs, s, f"{g}noise_res.{i}", 7, (1, 3, 5))
            else:
                xs = d.snake_resblock(d.conv(har_spec, f"{g}noise_convs.{i}"), s, f"{g}noise_res.{i}", 11, (1, 3, 5))
            x = F.conv_transpose1d(x, d.w[f"{g}ups.{i}.weight"], d.w.get(f"{g}ups.{i}.bias"), stride=rates[i], padding=(ksz[i] - rates[i]) // 2)
            if i == n_up - 1:
                x = torch.cat([x[:, :, 1:2], x], 2)                                       # reflection pad (1, 0)
            x = x + xs
            acc = 0
            for j, (k, dil) in enumerate(zip(ic["resblock_kernel_sizes"], ic["resblock_dilation_sizes"])):
                acc = acc + d.snake_resblock(x, s, f"{g}resblocks.{i * nk + j}", k, dil)
            x = acc / nk
        x = d.conv(F.leaky_relu(x, 0.01), g + "conv_post", padding=3)[0]
        bins = n_fft // 2 + 1
        return istft_small(torch.exp(x[:bins]), torch.sin(x[bins:]), n_fft, hop).cpu()


# ---- phonemisation ------------------------------------------------------------------------------------------------------
LETTER_SOUNDS = {"a": "æ", "b": "b", "c": "k", "d": "d", "e": "ɛ", "f": "f", "g": "ɡ", "h": "h", "i": "ɪ", "j": "ʤ", "k": "k",
                 "l": "l", "m": "m", "n": "n", "o": "ɑ", "p": "p", "q": "k", "r": "ɹ", "s": "s", "t": "t", "u": "ʌ", "v": "v",
                 "w": "w", "x": "ks", "y": "j", "z": "z"}
DIGRAPHS = {"th": "θ", "sh": "ʃ", "ch": "ʧ", "ng": "ŋ", "ph": "f", "ee": "i", "oo": "u", "ou": "W", "ow": "O", "ai": "A", "ay": "A",
            "oi": "Y", "oy": "Y", "ck": "k", "qu": "kw", "wh": "w"}


class KokoroG2p:
    """Word lookup in the snapshot's lexicon, letter-to-sound for the rest; punctuation Kokoro knows passes through."""

    def __init__(self, lexicon: dict[str, str] | None, vocab: dict):
        self.lex, self.vocab = lexicon or {}, vocab

    def word(self, w: str) -> str:
        lw = w.lower()
        if lw in self.lex:
            return self.lex[lw]
        out, i = [], 0
        while i < len(lw):
            if lw[i:i + 2] in DIGRAPHS:
                out.append(DIGRAPHS[lw[i:i + 2]])
                i += 2
            else:
                out.append(LETTER_SOUNDS.get(lw[i], ""))
                i += 1
        return "".join(out)

    def phonemize(self, text: str) -> str:
        if any(not c.isascii() for c in text):
            return text                                      # already a phoneme string (symbols outside the vocabulary drop out later)
        parts = []
        for tok in re.findall(r"[A-Za-z']+|[^A-Za-z'\s]+|\s+", text):
            if tok[0].isalpha() or tok[0] == "'":
                parts.append(self.word(tok.replace("'", "")))
            elif tok.isspace():
                parts.append(" ")
            else:
                parts.append("".join(c for c in tok if c in self.vocab))
        return "".join(parts).strip()


# ---- generator ----------------------------------------------------------------------------------------------------------
def kokoro_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family="kokoro", backend=backend, modality=Modality.AUDIO,
        capabilities=Capabilities(
            supports_negative_prompt=False, supports_guidance=False, supports_true_cfg=False, conditioning=[],
            supports_lora=False, supports_lokr=False, samplers=[], schedulers=[], supported_guidance_methods=[],
            min_size=0, max_size=0, max_count=1, audio_sample_rates=[SAMPLE_RATE], max_audio_duration_secs=MAX_DURATION_SECS,
            audio_voices=list(VOICES), audio_languages=list(LANGUAGES)),
        required_components=[])


def load_sections(root: Path) -> dict[str, dict[str, torch.Tensor]]:
    pth, st = root / CHECKPOINT_FILE, root / "kokoro.safetensors"
    if st.is_file():
        from ..io.safetensors_io import load_file

        out: dict[str, dict[str, torch.Tensor]] = {}
        for k, v in load_file(st).items():
            sec, _, name = k.partition(".")
            out.setdefault(sec, {})[name] = v
        return out
    if pth.is_file():
        return torch.load(pth, map_location="cpu", weights_only=True)
    raise LoadError(f"kokoro snapshot {root} has no {CHECKPOINT_FILE} (or kokoro.safetensors)")


class KokoroGenerator(Generator):
    def __init__(self, root: Path, backend: str, prefix: str = ""):
        self.root, self.backend = Path(root), backend
        self._descriptor = kokoro_descriptor(backend, prefix)
        self._pipe: KokoroPipeline | None = None
        self._voices: dict[str, torch.Tensor] = {}
        self._g2p: dict[str, KokoroG2p] = {}

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        if not req.prompt.strip():
            raise InferenceError(f"{mid}: prompt (the script text) must not be empty")
        self._descriptor.capabilities.validate_request_audio(mid, req)

    def pipeline(self) -> KokoroPipeline:
        if self._pipe is None:
            cj = self.root / "config.json"
            if not cj.is_file():
                raise LoadError(f"kokoro snapshot {self.root} has no config.json")
            cfg = KokoroConfig.from_json(json.loads(cj.read_text(encoding="utf-8")))
            dev = "cuda" if self.backend == "b200" else "cpu"
            self._pipe = KokoroPipeline(cfg, load_sections(self.root), dev)
        return self._pipe

    def voice_pack(self, voice: str) -> torch.Tensor:
        if voice not in self._voices:
            for ext in (".pt", ".safetensors"):
                f = self.root / "voices" / (voice + ext)
                if f.is_file():
                    if ext == ".pt":
                        t = torch.load(f, map_location="cpu", weights_only=True)
                    else:
                        from ..io.safetensors_io import load_file

                        t = next(iter(load_file(f).values()))
                    self._voices[voice] = t.float().reshape(t.shape[0], -1)
                    break
            else:
                raise InferenceError(f"{self._descriptor.id}: voice pack voices/{voice}.pt missing from the snapshot")
        return self._voices[voice]

    def g2p(self, british: bool) -> KokoroG2p:
        key = "gb" if british else "us"
        if key not in self._g2p:
            lex = self.root / "g2p" / f"{key}.json"
            self._g2p[key] = KokoroG2p(json.loads(lex.read_text(encoding="utf-8")) if lex.is_file() else None, self.pipeline().cfg.vocab)
        return self._g2p[key]

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        self.validate(req)
        if req.cancel.is_cancelled():
            raise Canceled(f"{self._descriptor.id}: cancelled")
        a = req.audio
        voice = (a.voice if a and a.voice else DEFAULT_VOICE)
        british = voice.startswith("b") or (not voice.startswith("a") and a is not None and a.language == "en-gb")
        pipe = self.pipeline()
        tokens = pipe.cfg.phonemes_to_ids(self.g2p(british).phonemize(req.prompt))
        if not tokens:
            raise InferenceError(f"{self._descriptor.id}: no phonemes survived tokenization (unsupported script?)")
        pack = self.voice_pack(voice)
        ref_s = pack[min(len(tokens), pack.shape[0]) - 1][None]
        speed = 1.0
        if a is not None and a.target_duration is not None and a.target_duration > 0:
            natural = pipe.natural_duration_secs(pipe.raw_durations(tokens, ref_s))
            speed = min(max(natural / a.target_duration, 0.5), 2.0)
        from ..media.seed import default_seed

        def stage(i: int):
            if i == STAGES - 1:
                on_progress(ProgressDecoding())
            on_progress(ProgressStep(i, STAGES))
            if req.cancel.is_cancelled():
                raise Canceled(f"{self._descriptor.id}: cancelled at stage {i}")

        samples = pipe.synthesize(tokens, ref_s, speed, req.seed if req.seed is not None else default_seed(), stage)
        secs = samples.numel() / SAMPLE_RATE
        if secs > 4.0 * MAX_DURATION_SECS:
            raise InferenceError(f"{self._descriptor.id}: predicted {secs:.1f}s exceeds the sane bound - refusing")
        return GenerationOutput(audio=AudioTrack(SAMPLE_RATE, 1, samples.tolist()))


def registration(backend: str) -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> KokoroGenerator:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise LoadError(f"{mid} expects a snapshot directory (config.json + {CHECKPOINT_FILE} + voices/), not a single file")
        if spec.quantize is not None:
            raise Unsupported(f"{mid} does not support on-the-fly quantization")
        if spec.adapters:
            raise Unsupported(f"{mid} does not support LoRA/LoKr adapters")
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid} does not support control/IP-adapter overlays")
        return KokoroGenerator(Path(spec.weights.path), backend, prefix)

    return Registration(descriptor=lambda: kokoro_descriptor(backend, prefix), load=load)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random Kokoro-shaped snapshot (safetensors sections, two voices, a four-word lexicon)."""
    from ..io.safetensors_io import save_file

    root = Path(root)
    (root / "voices").mkdir(parents=True, exist_ok=True)
    (root / "g2p").mkdir(exist_ok=True)
    H, S, W = 16, 8, 32
    vocab = {c: i + 1 for i, c in enumerate(" ,.!?abdefhijklmnpstuvwzæɛɪɑʌɹθʃʧŋʤɡAOWY")}
    cfg = dict(hidden_dim=H, style_dim=S, max_dur=6, n_layer=2, n_token=len(vocab) + 1, text_encoder_kernel_size=5,
               decoder_width=W,
               plbert=dict(hidden_size=24, num_attention_heads=2, intermediate_size=32, max_position_embeddings=64, num_hidden_layers=2),
               istftnet=dict(upsample_kernel_sizes=[20, 12], upsample_rates=[10, 6], gen_istft_hop_size=5, gen_istft_n_fft=20,
                             resblock_dilation_sizes=[[1, 3, 5], [1, 3, 5]], resblock_kernel_sizes=[3, 7], upsample_initial_channel=16),
               vocab=vocab)
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)      # noqa: E731
    w: dict[str, torch.Tensor] = {}

    def lin(p, o, i):
        w[p + ".weight"], w[p + ".bias"] = rn(o, i) / math.sqrt(i), rn(o) * 0.02

    def conv(p, o, i, k, bias=True, wn=False):
        t = rn(o, i, k) / math.sqrt(i * k)
        if wn:                                            # stored weight-normalised, as the published vocoder is
            w[p + ".weight_v"], w[p + ".weight_g"] = t, t.reshape(o, -1).norm(dim=1).reshape(o, 1, 1) * 1.0
        else:
            w[p + ".weight"] = t
        if bias:
            w[p + ".bias"] = rn(o) * 0.02

    def lstm(p, i, h):
        for sfx in ("", "_reverse"):
            w[f"{p}.weight_ih_l0{sfx}"], w[f"{p}.weight_hh_l0{sfx}"] = rn(4 * h, i) / math.sqrt(i), rn(4 * h, h) / math.sqrt(h)
            w[f"{p}.bias_ih_l0{sfx}"], w[f"{p}.bias_hh_l0{sfx}"] = rn(4 * h) * 0.02, rn(4 * h) * 0.02

    def resblk(p, i, o, up=False):
        lin(p + ".norm1.fc", 2 * i, S); lin(p + ".norm2.fc", 2 * o, S)      # noqa: E702
        conv(p + ".conv1", o, i, 3); conv(p + ".conv2", o, o, 3)      # noqa: E702
        if i != o:
            conv(p + ".conv1x1", o, i, 1, bias=False)
        if up:
            w[p + ".pool.weight"], w[p + ".pool.bias"] = rn(i, 1, 3) * 0.5, rn(i) * 0.02

    def snake(p, c, k, dil):
        for j in range(len(dil)):
            conv(f"{p}.convs1.{j}", c, c, k, wn=True); conv(f"{p}.convs2.{j}", c, c, k, wn=True)      # noqa: E702
            lin(f"{p}.adain1.{j}.fc", 2 * c, S); lin(f"{p}.adain2.{j}.fc", 2 * c, S)      # noqa: E702
            w[f"{p}.alpha1.{j}"], w[f"{p}.alpha2.{j}"] = torch.ones(1, c, 1), torch.ones(1, c, 1)

    pb = cfg["plbert"]
    b = "bert."
    w[b + "embeddings.word_embeddings.weight"] = rn(cfg["n_token"], 128) * 0.1
    w[b + "embeddings.position_embeddings.weight"] = rn(pb["max_position_embeddings"], 128) * 0.1
    w[b + "embeddings.token_type_embeddings.weight"] = rn(2, 128) * 0.1
    w[b + "embeddings.LayerNorm.weight"], w[b + "embeddings.LayerNorm.bias"] = torch.ones(128), torch.zeros(128)
    lin(b + "encoder.embedding_hidden_mapping_in", pb["hidden_size"], 128)
    L = b + "encoder.albert_layer_groups.0.albert_layers.0"
    for n in ("query", "key", "value", "dense"):
        lin(f"{L}.attention.{n}", pb["hidden_size"], pb["hidden_size"])
    lin(L + ".ffn", pb["intermediate_size"], pb["hidden_size"]); lin(L + ".ffn_output", pb["hidden_size"], pb["intermediate_size"])      # noqa: E702
    for n in (".attention.LayerNorm", ".full_layer_layer_norm"):
        w[L + n + ".weight"], w[L + n + ".bias"] = torch.ones(pb["hidden_size"]), torch.zeros(pb["hidden_size"])
    w["bert_encoder.weight"], w["bert_encoder.bias"] = rn(H, pb["hidden_size"]) / math.sqrt(pb["hidden_size"]), rn(H) * 0.02
    p = "predictor."
    for layer in range(cfg["n_layer"]):
        lstm(f"{p}text_encoder.lstms.{2 * layer}", H + S, H // 2)
        lin(f"{p}text_encoder.lstms.{2 * layer + 1}.fc", 2 * H, S)
    lstm(p + "lstm", H + S, H // 2); lstm(p + "shared", H + S, H // 2)      # noqa: E702
    lin(p + "duration_proj.linear_layer", cfg["max_dur"], H)
    for nm in ("F0", "N"):
        resblk(f"{p}{nm}.0", H, H); resblk(f"{p}{nm}.1", H, H // 2, up=True); resblk(f"{p}{nm}.2", H // 2, H // 2)      # noqa: E702
        conv(f"{p}{nm}_proj", 1, H // 2, 1)
    t = "text_encoder."
    w[t + "embedding.weight"] = rn(cfg["n_token"], H) * 0.3
    for i in range(cfg["n_layer"]):
        conv(f"{t}cnn.{i}.0", H, H, 5, wn=True)
        w[f"{t}cnn.{i}.1.gamma"], w[f"{t}cnn.{i}.1.beta"] = torch.ones(H), torch.zeros(H)
    lstm(t + "lstm", H, H // 2)
    d = "decoder."
    resblk(d + "encode", H + 2, W)
    for i in range(3):
        resblk(f"{d}decode.{i}", W + 2 + 8, W)
    resblk(d + "decode.3", W + 2 + 8, 16, up=True)
    conv(d + "F0_conv", 1, 1, 3, wn=True); conv(d + "N_conv", 1, 1, 3, wn=True); conv(d + "asr_res.0", 8, H, 1, wn=True)      # noqa: E702
    ic = cfg["istftnet"]
    gch = ic["upsample_initial_channel"]
    gp = d + "generator."
    w[gp + "m_source.l_linear.weight"], w[gp + "m_source.l_linear.bias"] = rn(1, 9) * 0.3, torch.zeros(1)
    for i, (u, k) in enumerate(zip(ic["upsample_rates"], ic["upsample_kernel_sizes"])):
        ci, co = gch // (1 << i), gch // (1 << (i + 1))
        tv = rn(ci, co, k) / math.sqrt(ci * k)
        w[f"{gp}ups.{i}.weight_v"], w[f"{gp}ups.{i}.weight_g"], w[f"{gp}ups.{i}.bias"] = tv, tv.reshape(ci, -1).norm(dim=1).reshape(ci, 1, 1), rn(co) * 0.02
        for j, (rk, rd) in enumerate(zip(ic["resblock_kernel_sizes"], ic["resblock_dilation_sizes"])):
            snake(f"{gp}resblocks.{i * len(ic['resblock_kernel_sizes']) + j}", co, rk, rd)
        if i + 1 < len(ic["upsample_rates"]):
            sf = math.prod(ic["upsample_rates"][i + 1:])
            conv(f"{gp}noise_convs.{i}", co, 22, sf * 2)
            snake(f"{gp}noise_res.{i}", co, 7, (1, 3, 5))
        else:
            conv(f"{gp}noise_convs.{i}", co, 22, 1)
            snake(f"{gp}noise_res.{i}", co, 11, (1, 3, 5))
    conv(gp + "conv_post", 22, gch // (1 << len(ic["upsample_rates"])), 7, wn=True)
    save_file({k: v.contiguous() for k, v in w.items()}, root / "kokoro.safetensors")
    (root / "config.json").write_text(json.dumps(cfg, ensure_ascii=False), encoding="utf-8")
    for i, v in enumerate(("af_heart", "bf_emma")):
        save_file({"pack": torch.randn(510, 1, 2 * S, generator=torch.Generator().manual_seed(seed + 10 + i)) * 0.3},
                  root / "voices" / f"{v}.safetensors")
    (root / "g2p" / "us.json").write_text(json.dumps({"hello": "həlO", "world": "wɜɹld", "the": "ðə", "fox": "fɑks"}, ensure_ascii=False),
                                          encoding="utf-8")
    return root
