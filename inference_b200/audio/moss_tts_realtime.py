"""MOSS-TTS-Realtime (`moss_tts_realtime`): streaming, context-aware text-to-speech at 24 kHz.

A Qwen3 backbone reads one multi-channel token per position (a text id plus `rvq` audio codebook ids, embedded and
summed); after each position a small depth transformer, seeded by the backbone's last hidden state, samples that frame's
`rvq` residual codebook tokens one after another; the frame is fed back as the next position's audio channels while the
remaining text streams in on the text channel. The MOSS-Audio-Tokenizer codec (a separate checkpoint, passed in as the
`codec` component) turns the frames into a waveform and, in the other direction, turns a reference clip or a
conversation turn's audio into frames.

Behaviour follows the reference's candle-audio-moss-tts-realtime crate:
  - config.rs:10-120         the backbone / depth-transformer configuration and its cross-checks
  - backbone.rs:20-215       summed channel embeddings, cached prefill and single-frame steps
  - local.rs:20-149          the depth transformer: rvq - 1 token tables, rvq heads, one sampled token per codebook
  - sampling.rs:5-230        repetition penalty over the last 50 tokens of the codebook, temperature, top-k, top-p,
                             inverse-CDF draw from a SplitMix64 stream
  - decode.rs:10-330         the system prompt with the optional voice-clone span, the 12-token text delay, the
                             generate / replay loops
  - conversation.rs:10-300   user / assistant turn layout on one growing cache, per-turn seeds
  - codec.rs:60-1230         residual lookup-free quantiser decode / encode, four causal banded-attention transformer
                             stages with channel-to-time patching, linear resampling of foreign sample rates
  - chunk.rs:10-110          streaming: every block of frames re-decodes the prefix and emits the new samples
  - model.rs:20-700          descriptor, request validation, generate / generate_streaming / conversation sessions

The backbone and depth transformer run on `OracleLlama` (fp32 on the oracle backend, bf16 tensor ops on a CUDA device)
because their inputs are summed embeddings, not token ids; the codec's projections run through `models.nn_dual` (the
tcgen05 GEMM on the device).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from pathlib import Path

import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, ConversationSession, ConversationTurn,
                                            GenerationOutput, GenerationRequest, Generator, Modality, ModelDescriptor)
from ..contracts.gen_core.license import WeightLicense
from ..contracts.gen_core.media import AudioChunk, AudioTrack
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec, ProgressDecoding, ProgressStep
from ..contracts.gen_core.traits import reject_unknown_components, require_component
from ..models import nn_dual as nd
from .moss_ttsd import Rng
from .moss_ttsd import sample as _draw

MODEL_ID = FAMILY = "moss_tts_realtime"
SAMPLE_RATE, FRAME_RATE_HZ = 24_000, 12.5
MAX_DURATION_SECS, DEFAULT_SECONDS, DEFAULT_SAMPLING_SEED = 2400.0, 10.0, 13_392
LANGUAGES = ["en", "zh"]
CODEC_COMPONENT_ID, MODEL_WEIGHTS = "codec", "model.safetensors"
DELAY_TOKENS_LEN = 12
DEFAULT_FRAMES_PER_BLOCK = 8
TEMPERATURE, TOP_P, TOP_K, REPETITION_PENALTY, REPETITION_WINDOW = 0.8, 0.6, 30, 1.1, 50
ASSISTANT_OPEN = "<|im_start|>assistant\n"
ASSISTANT_OPEN_AFTER_TURN = "<|im_end|>\n<|im_start|>assistant\n"
USER_OPEN = "<|im_end|>\n<|im_start|>user\n"
VOICE_CLONE_PREFIX = "<|im_start|>context\nThe assistant section should be synthesized using the following voice timbre:"
VOICE_CLONE_SUFFIX = "<|im_end|>\n"
AUDIO_PAD_STR, TEXT_PAD_STR = "<|audio_pad|>", "<|text_pad|>"
TTS_SYSTEM_PROMPT = ("<|im_start|>system\nYou are a highly expressive text-to-speech (TTS) engine developed by Mosi Intelligence. \n"
                     "You possess natural language understanding, emotional modeling, and multi-style speech generation "
                     "capabilities, allowing you to generate the corresponding speech based on the text given in the "
                     "assistant.<|im_end|>\n")
MOSS_TTS_REALTIME_LICENSE = WeightLicense("Apache-2.0", "Apache License 2.0", "https://huggingface.co/OpenMOSS-Team/MOSS-TTS-Realtime",
                                          "MOSS-TTS-Realtime-1.7B (c) OpenMOSS Team - licensed under Apache-2.0", True)


# ---- configuration ----------------------------------------------------------------------------------------------------------
@dataclass
class RealtimeConfig:
    language: dict
    local: dict
    rvq: int
    audio_vocab_size: int
    audio_pad_token: int
    text_pad: int = 151_655
    reference_audio_pad: int = 151_654

    @property
    def audio_bos(self) -> int:
        return self.audio_pad_token + 1

    @property
    def audio_eos(self) -> int:
        return self.audio_pad_token + 2

    @staticmethod
    def from_json(j: dict) -> "RealtimeConfig":
        for k in ("language_config", "local_config", "rvq", "audio_vocab_size", "audio_pad_token"):
            if k not in j:
                raise LoadError(f"{MODEL_ID}: config.json lacks {k}")
        cfg = RealtimeConfig(j["language_config"], j["local_config"], int(j["rvq"]), int(j["audio_vocab_size"]),
                             int(j["audio_pad_token"]), int(j.get("text_pad", 151_655)), int(j.get("reference_audio_pad", 151_654)))
        if cfg.rvq != int(cfg.local.get("rvq", cfg.rvq)):
            raise LoadError(f"{MODEL_ID}: config.json rvq ({cfg.rvq}) disagrees with local_config.rvq ({cfg.local.get('rvq')})")
        if cfg.rvq <= 0:
            raise LoadError(f"{MODEL_ID}: config.json rvq must be > 0")
        if cfg.audio_eos >= cfg.audio_vocab_size:
            raise LoadError(f"{MODEL_ID}: audio_vocab_size {cfg.audio_vocab_size} has no room for the begin / end tokens after "
                            f"audio_pad_token {cfg.audio_pad_token}")
        return cfg


def _llama_config(j: dict, vocab: int):
    from ..models.config import ModelConfig

    return ModelConfig.from_json({
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": vocab, "hidden_size": j["hidden_size"],
        "intermediate_size": j["intermediate_size"], "num_hidden_layers": j["num_hidden_layers"],
        "num_attention_heads": j["num_attention_heads"], "num_key_value_heads": j["num_key_value_heads"], "head_dim": j["head_dim"],
        "rms_norm_eps": j.get("rms_norm_eps", 1e-6), "rope_theta": j.get("rope_theta", 1e6),
        "attention_bias": j.get("attention_bias", False), "tie_word_embeddings": True, "max_position_embeddings": 65536})


# ---- sampling ---------------------------------------------------------------------------------------------------------------
@dataclass
class SamplingParams:
    temperature: float = TEMPERATURE
    top_p: float = TOP_P
    top_k: int = TOP_K
    repetition_penalty: float = REPETITION_PENALTY
    repetition_window: int = REPETITION_WINDOW

    @staticmethod
    def from_env() -> "SamplingParams":
        def num(key, default, cast):
            try:
                v = cast(os.environ[key].strip())
            except (KeyError, ValueError):
                return default
            return v if math.isfinite(v) else default
        return SamplingParams(num("MOSS_TTS_TEMPERATURE", TEMPERATURE, float), num("MOSS_TTS_TOP_P", TOP_P, float),
                              int(num("MOSS_TTS_TOP_K", TOP_K, int)), num("MOSS_TTS_REP_PENALTY", REPETITION_PENALTY, float))


def sample(logits: torch.Tensor, history: list[int], p: SamplingParams, rng: Rng) -> int:
    """Logits of one codebook (1-D fp32): tokens among the codebook's last `repetition_window` picks are pushed down
    (positive logits divided, negative multiplied), then temperature / top-k / top-p and one draw."""
    lg = logits.float().clone()
    if p.repetition_penalty != 1.0 and history:
        recent = torch.tensor(sorted({t for t in history[-p.repetition_window:] if t < lg.numel()}), dtype=torch.int64)
        if recent.numel():
            v = lg[recent]
            lg[recent] = torch.where(v < 0, v * p.repetition_penalty, v / p.repetition_penalty)
    return _draw(lg, rng, p.temperature, p.top_k, p.top_p)


def min_eos_frames(budget: int) -> int:
    """Frames during which the end token is suppressed (MOSS_TTS_MIN_FRAMES, default 0), never above half the budget."""
    try:
        n = int(os.environ.get("MOSS_TTS_MIN_FRAMES", "0").strip())
    except ValueError:
        n = 0
    return min(max(n, 0), budget // 2)


# ---- backbone and depth transformer -------------------------------------------------------------------------------------------
def _dtype_for(device: torch.device):
    return torch.bfloat16 if device.type == "cuda" else torch.float32


class Backbone:
    def __init__(self, cfg: RealtimeConfig, weights: dict[str, torch.Tensor], device="cpu"):
        from ..models.oracle import OracleLlama

        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = _dtype_for(self.device)
        self.tables = []
        for c in range(cfg.rvq + 1):
            k = f"embed_tokens.{c}.weight"
            if k not in weights:
                raise LoadError(f"{MODEL_ID}: checkpoint lacks {k}")
            self.tables.append(weights[k].to(self.device, self.dtype))
        lm = {"model." + k[len("language_model."):]: v for k, v in weights.items() if k.startswith("language_model.")}
        lm["model.embed_tokens.weight"] = weights["embed_tokens.0.weight"]
        self.lm = OracleLlama(_llama_config(cfg.language, self.tables[0].shape[0]), lm, self.dtype, self.device)

    def new_cache(self):
        from ..models.oracle import ContiguousKvCache

        return ContiguousKvCache(int(self.cfg.language["num_hidden_layers"]))

    def embed(self, frames: list[list[int]]) -> torch.Tensor:
        """frames: rows of [text id, audio id x rvq] -> [1, T, hidden], the sum of the channel embeddings."""
        t = torch.tensor(frames, dtype=torch.int64, device=self.device)
        return sum(self.tables[c][t[:, c]] for c in range(self.cfg.rvq + 1))[None]

    @torch.no_grad()
    def forward(self, frames: list[list[int]], cache) -> torch.Tensor:
        """Appends `frames` to the cache -> the final-norm hidden state of the last position [1, 1, hidden]."""
        h = self.lm.hidden_states(None, cache, cache.offset, embeds=self.embed(frames))
        return self.lm._norm(h[:, -1:], "model.norm.weight")


class LocalTransformer:
    def __init__(self, cfg: RealtimeConfig, weights: dict[str, torch.Tensor], device="cpu"):
        from ..models.oracle import OracleLlama

        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = _dtype_for(self.device)
        pre = "local_transformer.model."
        lm = {"model." + k[len(pre):]: v for k, v in weights.items() if k.startswith(pre) and not k.startswith(pre + "embed_tokens.")}
        self.tables, self.heads = [], []
        for i in range(cfg.rvq):
            if i + 1 < cfg.rvq:
                k = f"{pre}embed_tokens.{i}.weight"
                if k not in weights:
                    raise LoadError(f"{MODEL_ID}: checkpoint lacks {k}")
                self.tables.append(weights[k].to(self.device, self.dtype))
            k = f"local_transformer.local_lm_heads.{i}.weight"
            if k not in weights:
                raise LoadError(f"{MODEL_ID}: checkpoint lacks {k}")
            self.heads.append(weights[k].to(self.device, self.dtype))
        lm["model.embed_tokens.weight"] = self.tables[0] if self.tables else self.heads[0]
        self.layers = int(cfg.local["num_hidden_layers"])
        self.lm = OracleLlama(_llama_config(cfg.local, lm["model.embed_tokens.weight"].shape[0]), lm, self.dtype, self.device)

    @torch.no_grad()
    def decode_frame(self, hidden: torch.Tensor, history: list[list[int]], p: SamplingParams, rng: Rng, suppress_eos: bool
                     ) -> list[int]:
        """One frame: position 0 of the depth sequence is the backbone's hidden state [1, 1, H], position i the
        embedding of codebook i - 1's token; codebook i is sampled from head i at position i."""
        from ..models.oracle import ContiguousKvCache

        cache = ContiguousKvCache(self.layers)
        x, tokens = hidden.to(self.dtype), []
        for i in range(self.cfg.rvq):
            h = self.lm._norm(self.lm.hidden_states(None, cache, cache.offset, embeds=x)[:, -1], "model.norm.weight")
            logits = (h @ self.heads[i].t()).float().cpu()[0]
            if i == 0 and suppress_eos:
                logits[self.cfg.audio_eos] = float("-inf")
            tok = sample(logits, [f[i] for f in history if i < len(f)], p, rng)
            tokens.append(tok)
            if i + 1 < self.cfg.rvq:
                x = self.tables[i][tok][None, None]
        return tokens


# ---- prompt layout ----------------------------------------------------------------------------------------------------------
def _ids(tokenizer, s: str) -> list[int]:
    return tokenizer.encode(s, add_special_tokens=False).ids


def pad_frame(cfg: RealtimeConfig, text_id: int) -> list[int]:
    return [text_id] + [cfg.audio_pad_token] * cfg.rvq


def system_frames(tokenizer, cfg: RealtimeConfig, reference: list[list[int]] | None) -> list[list[int]]:
    """The system prompt; with a reference clip, a context section whose audio-pad positions carry the clip's frames."""
    text = TTS_SYSTEM_PROMPT
    if reference:
        text += VOICE_CLONE_PREFIX + AUDIO_PAD_STR * len(reference) + VOICE_CLONE_SUFFIX
    frames, k = [], 0
    for tid in _ids(tokenizer, text):
        f = pad_frame(cfg, tid)
        if reference and tid == cfg.reference_audio_pad:
            if k >= len(reference):
                raise InferenceError(f"{MODEL_ID}: voice clone: audio-pad position {k} exceeds the reference frames")
            if len(reference[k]) != cfg.rvq:
                raise InferenceError(f"{MODEL_ID}: voice clone: reference frame {k} has {len(reference[k])} codes, expected {cfg.rvq}")
            f[1:] = reference[k]
            k += 1
        frames.append(f)
    if reference and k != len(reference):
        raise InferenceError(f"{MODEL_ID}: voice clone: {len(reference)} reference frames but {k} audio-pad positions")
    return frames


def assistant_prefill(tokenizer, cfg: RealtimeConfig, opener: str, text: str, frames: list[list[int]]) -> list[int]:
    """Appends the opener and the first DELAY_TOKENS_LEN text tokens to `frames` (the last of them carries the audio
    begin token on codebook 0) -> the text tokens that stream in during generation."""
    ids = _ids(tokenizer, text)
    if not ids:
        raise InferenceError(f"{MODEL_ID}: empty assistant text after tokenization")
    n = min(len(ids), DELAY_TOKENS_LEN)
    for tid in _ids(tokenizer, opener) + ids[:n]:
        frames.append(pad_frame(cfg, tid))
    frames[-1][1] = cfg.audio_bos
    return ids[n:]


def user_body_frames(tokenizer, cfg: RealtimeConfig, text: str, codes: list[list[int]]) -> list[list[int]]:
    """A user turn: its text on the text channel followed by text pads, its audio on the audio channels starting
    DELAY_TOKENS_LEN tokens into the text (or right after a shorter text), bracketed by begin / end on codebook 0."""
    if not codes:
        raise InferenceError(f"{MODEL_ID}: a user turn carries no audio")
    for i, row in enumerate(codes):
        if len(row) != cfg.rvq:
            raise InferenceError(f"{MODEL_ID}: user audio frame {i} has {len(row)} codes, expected {cfg.rvq}")
    start, n_text, n_audio = len(_ids(tokenizer, USER_OPEN)), len(_ids(tokenizer, text)), len(codes)
    if n_text == 0:
        raise InferenceError(f"{MODEL_ID}: empty user text")
    long = n_text >= DELAY_TOKENS_LEN
    pads = n_audio + DELAY_TOKENS_LEN - n_text + 1 if long else n_audio + 1
    frames = [pad_frame(cfg, t) for t in _ids(tokenizer, USER_OPEN + text + TEXT_PAD_STR * pads)]
    at = start + DELAY_TOKENS_LEN if long else len(frames) - (n_audio + 1)
    if at < 1 or at + n_audio >= len(frames):
        raise InferenceError(f"{MODEL_ID}: user audio span [{at}..{at + n_audio}] does not fit the {len(frames)}-token user body")
    for k, row in enumerate(codes):
        frames[at + k][1:] = row
    frames[at - 1][1] = cfg.audio_bos
    frames[at + n_audio][1] = cfg.audio_eos
    return frames


# ---- autoregressive loops ---------------------------------------------------------------------------------------------------
class Decoder:
    def __init__(self, cfg: RealtimeConfig, weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg = cfg
        self.backbone, self.local = Backbone(cfg, weights, device), LocalTransformer(cfg, weights, device)

    def generate_turn(self, cache, prefill: list[list[int]], streamed: list[int], max_frames: int, seed: int,
                      cancel=lambda: False, on_frame=lambda step, frame: None) -> tuple[list[list[int]], str] | None:
        """-> (frames, "eos" | "budget"); None when cancelled. Frame k + 1 is conditioned on frame k fed back with
        streamed text token k (the text pad once the text has run out)."""
        out: list[list[int]] = []
        params, rng, floor = SamplingParams.from_env(), Rng(seed), min_eos_frames(max_frames)
        for step in range(max_frames):
            if cancel():
                return None
            if step == 0:
                hidden = self.backbone.forward(prefill, cache)
            else:
                text = streamed[step - 1] if step - 1 < len(streamed) else self.cfg.text_pad
                hidden = self.backbone.forward([[text] + out[-1]], cache)
            frame = self.local.decode_frame(hidden, out, params, rng, len(out) < floor)
            if frame[0] == self.cfg.audio_eos:
                return out, "eos"
            if on_frame(step, frame) is False:
                return None
            out.append(frame)
        return out, "budget"

    def replay_turn(self, cache, prefill: list[list[int]], streamed: list[int], frames: list[list[int]], cancel=lambda: False) -> bool:
        """Advances the cache over an assistant turn whose audio is given; False when cancelled."""
        if cancel():
            return False
        self.backbone.forward(prefill, cache)
        for i, f in enumerate(frames):
            if cancel():
                return False
            self.backbone.forward([[streamed[i] if i < len(streamed) else self.cfg.text_pad] + list(f)], cache)
        return True


@dataclass
class PreparedTurn:
    role: str
    text: str
    codes: list[list[int]] | None = None


def turn_seed(base: int, ordinal: int) -> int:
    return (base + ordinal * 0x9E3779B97F4A7C15) & ((1 << 64) - 1)


class ConvState:
    def __init__(self, decoder: Decoder):
        self.cache, self.first, self.ordinal, self.after_turn = decoder.backbone.new_cache(), True, 0, False


def advance_turn(decoder: Decoder, tokenizer, reference, state: ConvState, turn: PreparedTurn, base_seed: int, budget: int,
                 cancel=lambda: False, on_frame=lambda step, frame: None) -> list[list[int]] | None:
    """One turn on the conversation's cache -> the turn's frames (given or generated); None when cancelled."""
    if cancel():
        return None
    cfg, block = decoder.cfg, []
    if state.first:
        block += system_frames(tokenizer, cfg, reference)
        state.first = False
    if turn.role == "user":
        if turn.codes is None:
            raise InferenceError(f"{MODEL_ID}: a user turn must carry its audio")
        block += user_body_frames(tokenizer, cfg, turn.text, turn.codes)
        decoder.backbone.forward(block, state.cache)
        state.after_turn = True
        return turn.codes
    streamed = assistant_prefill(tokenizer, cfg, ASSISTANT_OPEN_AFTER_TURN if state.after_turn else ASSISTANT_OPEN, turn.text, block)
    state.after_turn = True
    if turn.codes is not None:
        for i, row in enumerate(turn.codes):
            if len(row) != cfg.rvq:
                raise InferenceError(f"{MODEL_ID}: provided assistant frame {i} has {len(row)} codes, expected {cfg.rvq}")
        return turn.codes if decoder.replay_turn(state.cache, block, streamed, turn.codes, cancel) else None
    seed = turn_seed(base_seed, state.ordinal)
    state.ordinal += 1
    r = decoder.generate_turn(state.cache, block, streamed, budget, seed, cancel, on_frame)
    return None if r is None else r[0]


# ---- codec ------------------------------------------------------------------------------------------------------------------
HEAD_DIM, ROPE_MAX_PERIOD, LN_EPS = 64, 10_000.0, 1e-5
DECODER_PATCHES, ENCODER_PATCHES = (2, 2, 2, 240), (240, 2, 2, 2)


def fold_weight_norm_1x1(w: dict[str, torch.Tensor], p: str) -> tuple[torch.Tensor, torch.Tensor]:
    """A weight-normed kernel-1 convolution as (matrix [out, in], bias)."""
    g, v = w.get(p + ".parametrizations.weight.original0"), w.get(p + ".parametrizations.weight.original1")
    if g is None or v is None or p + ".bias" not in w:
        raise LoadError(f"{MODEL_ID} codec: missing tensors of {p}")
    v = v.float()
    return (v * g.float() / v.pow(2).sum(dim=(1, 2), keepdim=True).sqrt())[:, :, 0], w[p + ".bias"].float()


def band_mask(length: int, context: int, device) -> torch.Tensor:
    """Query i sees keys j with j <= i and i - j < context."""
    i = torch.arange(length, device=device)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < context)


def unpatch(x: torch.Tensor, p: int) -> torch.Tensor:
    """[B, D * p, L] -> [B, D, L * p]: the p channel groups of a position become p consecutive time steps."""
    B, C, L = x.shape
    if C % p:
        raise InferenceError(f"{MODEL_ID} codec: {C} channels not divisible by patch {p}")
    return x.reshape(B, C // p, p, L).permute(0, 1, 3, 2).reshape(B, C // p, L * p)


def patch(x: torch.Tensor, p: int) -> torch.Tensor:
    """The inverse: [B, D, L] -> [B, D * p, L / p]."""
    B, D, L = x.shape
    if L % p:
        raise InferenceError(f"{MODEL_ID} codec: length {L} not divisible by patch {p}")
    return x.reshape(B, D, L // p, p).permute(0, 1, 3, 2).reshape(B, D * p, L // p)


def resample_linear(x: torch.Tensor, src: int, dst: int) -> torch.Tensor:
    """1-D linear-interpolation resampling (output sample i reads source position i * src / dst)."""
    if src == dst or x.numel() == 0:
        return x
    n = max(int(round(x.numel() * dst / src)), 1)
    pos = torch.arange(n, dtype=torch.float64) * (src / dst)
    j = pos.floor().long()
    frac = (pos - j).float()
    last = x.numel() - 1
    a, b = x[j.clamp(max=last)], x[(j + 1).clamp(max=last)]
    return a + (b - a) * frac


class CodecStage:
    """A causal transformer over [1, C, T] features: optional input / output projections around pre-LayerNorm blocks with
    fused q/k/v, interleaved rotary phases, attention banded to `context` positions, erf-GELU MLP and learned
    per-channel residual scales."""

    def __init__(self, w: nd.WeightBag, prefix: str, context: int):
        self.w, self.p, self.context = w, prefix, max(context, 1)
        self.layers = 0
        while f"{prefix}transformer.layers.{self.layers}.norm1.weight" in w:
            self.layers += 1
        if self.layers == 0:
            raise LoadError(f"{MODEL_ID} codec: no transformer layers under {prefix}")
        self.d = w[f"{prefix}transformer.layers.0.norm1.weight"].shape[0]
        self.heads = max(self.d // HEAD_DIM, 1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, p = self.w, self.p
        h = x.transpose(1, 2).to(w.dtype)
        if p + "input_proj.weight" in w:
            h = nd.linear(h, w[p + "input_proj.weight"])
        T, H, D = h.shape[1], self.heads, self.d // self.heads
        inv = 1.0 / (ROPE_MAX_PERIOD ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
        cos, sin = ang.cos().float().to(h.device), ang.sin().float().to(h.device)
        mask = band_mask(T, self.context, h.device)
        for i in range(self.layers):
            b = f"{p}transformer.layers.{i}."
            y = nd.layer_norm(h, w[b + "norm1.weight"], w[b + "norm1.bias"], LN_EPS)
            qkv = nd.linear(y, w[b + "self_attn.in_projs.0.weight"]).view(1, T, 3, H, D)
            q, k = nd.rope_interleaved(qkv[:, :, 0], cos, sin), nd.rope_interleaved(qkv[:, :, 1], cos, sin)
            a = nd.linear(nd.attention(q, k, qkv[:, :, 2], mask=mask), w[b + "self_attn.out_projs.0.weight"])
            h = h + a * w[b + "layer_scale_1.scale"]
            y = nd.layer_norm(h, w[b + "norm2.weight"], w[b + "norm2.bias"], LN_EPS)
            y = nd.linear(nd.linear(y, w[b + "linear1.weight"], act="gelu"), w[b + "linear2.weight"])
            h = h + y * w[b + "layer_scale_2.scale"]
        if p + "output_proj.weight" in w:
            h = nd.linear(h, w[p + "output_proj.weight"])
        return h.transpose(1, 2)


class MossAudioCodec:
    """MOSS-Audio-Tokenizer: frames of residual codes <-> 24 kHz mono waveform. `nq` = codebooks in use (the first `nq` of
    the codec's quantisers: its variable-bitrate decode)."""

    def __init__(self, root: Path, nq: int, device="cpu"):
        from ..io.safetensors_io import load_file

        root = Path(root)
        cj = root / "config.json"
        if not cj.is_file():
            raise LoadError(f"{MODEL_ID} codec: {cj} missing")
        j = json.loads(cj.read_text(encoding="utf-8"))
        arch = j.get("architectures") or []
        if arch and "MossAudioTokenizerModel" not in arch:
            raise LoadError(f"{MODEL_ID} codec: architectures {arch} is not MossAudioTokenizerModel")
        q = j.get("quantizer_kwargs", {})
        qtype = q.get("quantizer_type") or j.get("quantizer_type") or "rvq"
        if qtype not in ("rlfq", "random_prefix_rlfq"):
            raise LoadError(f"{MODEL_ID} codec: quantizer_type {qtype!r} is not the residual lookup-free quantiser this decoder implements")
        self.sample_rate = int(j.get("sample_rate") or SAMPLE_RATE)
        self.hop = int(j["downsample_rate"])
        self.dec_patches = tuple(j.get("decoder_patch_sizes") or DECODER_PATCHES)
        self.enc_patches = tuple(j.get("encoder_patch_sizes") or ENCODER_PATCHES)
        if math.prod(self.dec_patches) != self.hop or math.prod(self.enc_patches) != self.hop:
            raise LoadError(f"{MODEL_ID} codec: patch sizes {self.dec_patches} / {self.enc_patches} do not multiply to downsample_rate {self.hop}")
        self.context_secs = float(j.get("causal_transformer_context_duration", 10.0))
        self.num_quantizers, self.codebook_size = int(q["num_quantizers"]), int(q["codebook_size"])
        if nq <= 0 or nq > self.num_quantizers:
            raise LoadError(f"{MODEL_ID} codec: requested {nq} quantisers, the codec has {self.num_quantizers}")
        self.nq, self.device = nq, torch.device(device)
        files = sorted(f for f in root.glob("model*.safetensors"))
        if not files:
            raise LoadError(f"{MODEL_ID} codec: no model*.safetensors in {root}")
        raw: dict[str, torch.Tensor] = {}
        for f in files:
            raw.update(load_file(f))
        self.raw = {k: v for k, v in raw.items() if k.startswith("quantizer.")}
        self.w = nd.WeightBag({k: v for k, v in raw.items() if k.startswith(("decoder.", "encoder."))}, _dtype_for(self.device), self.device)
        dev = self.device
        self.codebooks = [raw[f"quantizer.quantizers.{i}.codebook.weight"].float().to(dev) for i in range(nq)]
        self.out_projs = [tuple(t.to(dev) for t in fold_weight_norm_1x1(raw, f"quantizer.quantizers.{i}.out_proj")) for i in range(nq)]
        self.output_proj = tuple(t.to(dev) for t in fold_weight_norm_1x1(raw, "quantizer.output_proj"))
        self.stages, rate = [], self.sample_rate / self.hop
        for si, pz in enumerate(self.dec_patches):
            self.stages.append(CodecStage(self.w, f"decoder.{2 * si}.", int(rate * self.context_secs)))
            rate *= pz
        self._encoder = None

    # -- decode --
    @torch.no_grad()
    def decode_frames(self, frames: list[list[int]], cancel=lambda: False) -> torch.Tensor | None:
        """frames [T][nq] -> waveform [T * hop] on the host; None when cancelled."""
        if not frames:
            return torch.zeros(0)
        if cancel():
            return None
        codes = torch.tensor([[f[q] if q < len(f) else 0 for q in range(self.nq)] for f in frames], dtype=torch.int64,
                             device=self.device).clamp_(max=self.codebook_size - 1)
        emb = 0
        for q in range(self.nq):
            wq, bq = self.out_projs[q]
            emb = emb + self.codebooks[q][codes[:, q]] @ wq.t() + bq
        x = (emb @ self.output_proj[0].t() + self.output_proj[1]).t()[None]                     # [1, code dim, T]
        for stage, pz in zip(self.stages, self.dec_patches):
            if cancel():
                return None
            x = unpatch(stage.forward(x).float(), pz)
        return x[0, 0].float().cpu()

    # -- encode --
    def _encoder_half(self):
        if self._encoder is None:
            raw, dev = self.raw, self.device
            stages, rate = [], float(self.sample_rate)
            for si, pz in enumerate(self.enc_patches):
                rate /= pz
                stages.append(CodecStage(self.w, f"encoder.{2 * si + 1}.", int(rate * self.context_secs)))
            inp = tuple(t.to(dev) for t in fold_weight_norm_1x1(raw, "quantizer.input_proj"))
            ins = [tuple(t.to(dev) for t in fold_weight_norm_1x1(raw, f"quantizer.quantizers.{i}.in_proj")) for i in range(self.nq)]
            self._encoder = (stages, inp, ins)
        return self._encoder

    @torch.no_grad()
    def encode(self, samples: torch.Tensor, sample_rate: int) -> list[list[int]]:
        """mono waveform -> frames [floor(T / hop)][nq]: each stage patches time into channels and runs its transformer;
        each quantiser picks the codebook row with the largest cosine similarity to its projection of the residual."""
        wav = resample_linear(samples.float().reshape(-1), sample_rate, self.sample_rate)
        valid = wav.numel() // self.hop
        if valid == 0:
            return []
        stages, inp, ins = self._encoder_half()
        x = F.pad(wav, (0, (-wav.numel()) % self.hop)).to(self.device)[None, None]
        for stage, pz in zip(stages, self.enc_patches):
            x = stage.forward(patch(x.float(), pz))
        residual = x[0].float().t() @ inp[0].t() + inp[1]                                      # [T, rvq dim]
        rows = []
        for q in range(self.nq):
            z = F.normalize(residual @ ins[q][0].t() + ins[q][1], dim=1, eps=1e-12)
            idx = (z @ F.normalize(self.codebooks[q], dim=1, eps=1e-12).t()).argmax(dim=1)
            residual = residual - (self.codebooks[q][idx] @ self.out_projs[q][0].t() + self.out_projs[q][1])
            rows.append(idx.cpu().tolist())
        return [[rows[q][t] for q in range(self.nq)] for t in range(valid)]


class StreamingChunker:
    """Every `block` frames the whole prefix is decoded again (the codec is causal, so earlier samples do not change) and
    the samples past what was already emitted go out as the next chunk."""

    def __init__(self, codec, block: int, on_chunk=lambda c: None):
        self.codec, self.block, self.on_chunk = codec, max(block, 1), on_chunk
        self.frames: list[list[int]] = []
        self.samples = torch.zeros(0)
        self.flushed, self.index = 0, 0

    def push(self, frame: list[int], cancel=lambda: False) -> bool:
        self.frames.append(list(frame))
        return self._flush(cancel) if len(self.frames) % self.block == 0 else True

    def finish(self, cancel=lambda: False) -> torch.Tensor | None:
        if self.flushed != len(self.frames) and not self._flush(cancel):
            return None
        return self.samples

    def _flush(self, cancel) -> bool:
        pcm = self.codec.decode_frames(self.frames, cancel)
        if pcm is None:
            return False
        self.flushed = len(self.frames)
        tail = pcm[min(self.samples.numel(), pcm.numel()):]
        if tail.numel():
            self.on_chunk(AudioChunk(self.codec.sample_rate, 1, tail.tolist(), self.index))
            self.samples = torch.cat([self.samples, tail])
            self.index += 1
        return True


# ---- generator --------------------------------------------------------------------------------------------------------------
def moss_tts_realtime_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family=FAMILY, backend=backend, modality=Modality.AUDIO,
        capabilities=Capabilities(
            supports_negative_prompt=False, supports_guidance=False, supports_true_cfg=False,
            conditioning=[ConditioningKind.REFERENCE_AUDIO, ConditioningKind.CONVERSATION_HISTORY], supports_lora=False,
            supports_lokr=False, samplers=[], schedulers=[], supported_guidance_methods=[], min_size=0, max_size=0, max_count=1,
            audio_sample_rates=[SAMPLE_RATE], max_audio_duration_secs=MAX_DURATION_SECS, audio_voices=[],
            audio_languages=list(LANGUAGES), supports_streaming=True, supports_conversation_history=True,
            supports_conversation_session=True),
        required_components=[CODEC_COMPONENT_ID])


def frame_budget(req: GenerationRequest) -> int:
    a = req.audio
    secs = a.target_duration if a is not None and a.target_duration is not None else DEFAULT_SECONDS
    return max(int(math.ceil(secs * FRAME_RATE_HZ)), 1)


def frames_per_block(budget: int) -> int:
    return max(min(DEFAULT_FRAMES_PER_BLOCK, -(-budget // 2)), 1)


def mono(track: AudioTrack) -> torch.Tensor:
    x = torch.tensor(track.samples, dtype=torch.float32)
    ch = max(track.channels, 1)
    return x if ch == 1 else x[: x.numel() // ch * ch].view(-1, ch).mean(dim=1)


def _conditioning(req: GenerationRequest, kind: ConditioningKind):
    return next((c for c in req.conditioning if c.kind is kind), None)


class MossTtsRealtimeGenerator(Generator):
    def __init__(self, root: Path, codec_dir: Path, backend: str, prefix: str = ""):
        self.root, self.codec_dir, self.backend = Path(root), Path(codec_dir), backend
        self._descriptor = moss_tts_realtime_descriptor(backend, prefix)
        self._loaded = None
        self._codec: MossAudioCodec | None = None

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def _device(self) -> str:
        return "cuda" if self.backend == "b200" else "cpu"

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        if _conditioning(req, ConditioningKind.CONVERSATION_HISTORY) is None and not req.prompt.strip():
            raise InferenceError(f"{mid}: prompt (the text to speak) must not be empty")
        self._descriptor.capabilities.validate_request_audio(mid, req)

    def pipeline(self):
        if self._loaded is None:
            import tokenizers

            from ..io.safetensors_io import load_file

            cj, tk, wf = self.root / "config.json", self.root / "tokenizer.json", self.root / MODEL_WEIGHTS
            for f in (cj, tk, wf):
                if not f.is_file():
                    raise LoadError(f"{MODEL_ID}: {f} missing (the snapshot must supply config.json, tokenizer.json and {MODEL_WEIGHTS})")
            cfg = RealtimeConfig.from_json(json.loads(cj.read_text(encoding="utf-8")))
            self._loaded = (Decoder(cfg, load_file(wf), self._device()), tokenizers.Tokenizer.from_file(str(tk)))
        return self._loaded

    def codec(self) -> MossAudioCodec:
        if self._codec is None:
            self._codec = MossAudioCodec(self.codec_dir, self.pipeline()[0].cfg.rvq, self._device())
        return self._codec

    def _encode_track(self, track: AudioTrack, what: str) -> list[list[int]]:
        codec = self.codec()
        codes = codec.encode(mono(track), track.sample_rate)
        if not codes:
            raise InferenceError(f"{MODEL_ID}: {what} too short to encode (needs >= {codec.hop} samples at {codec.sample_rate} Hz)")
        return codes

    def reference_codes(self, req: GenerationRequest) -> list[list[int]] | None:
        c = _conditioning(req, ConditioningKind.REFERENCE_AUDIO)
        if c is None:
            return None
        if c.audio is None or not c.audio.samples:
            raise InferenceError(f"{MODEL_ID}: reference audio conditioning carries no samples")
        return self._encode_track(c.audio, "reference audio")

    def prepare_turn(self, turn: ConversationTurn, index: int) -> PreparedTurn:
        codes = self._encode_track(turn.audio, f"conversation turn {index} audio") if turn.audio is not None else None
        return PreparedTurn(turn.role, turn.text, codes)

    def rvq_frames(self, req: GenerationRequest, on_progress=lambda p: None, on_frame=lambda f: True) -> tuple[list[list[int]], str]:
        """The autoregressive half of a single-utterance request -> (frames, "eos" | "budget")."""
        self.validate(req)
        if req.cancel.is_cancelled():
            raise Canceled(f"{MODEL_ID}: cancelled")
        decoder, tokenizer = self.pipeline()
        prefill = system_frames(tokenizer, decoder.cfg, self.reference_codes(req))
        streamed = assistant_prefill(tokenizer, decoder.cfg, ASSISTANT_OPEN, req.prompt, prefill)
        budget = frame_budget(req)

        def frame_cb(step, frame):
            on_progress(ProgressStep(step + 1, budget))
            return on_frame(frame)

        r = decoder.generate_turn(decoder.backbone.new_cache(), prefill, streamed, budget,
                                  req.seed if req.seed is not None else DEFAULT_SAMPLING_SEED, req.cancel.is_cancelled, frame_cb)
        if r is None:
            raise Canceled(f"{MODEL_ID}: cancelled")
        return r

    def _synthesize(self, req: GenerationRequest, on_progress, on_chunk) -> AudioTrack:
        hist = _conditioning(req, ConditioningKind.CONVERSATION_HISTORY)
        if hist is not None:
            self.validate(req)
            if req.cancel.is_cancelled():
                raise Canceled(f"{MODEL_ID}: cancelled")
            session = self.open_conversation(req)
            total = max(sum(1 for t in hist.turns if t.role == "assistant" and t.audio is None), 1) * session.budget
            count, parts, index = [0], [], [0]

            def progress(p):
                if isinstance(p, ProgressStep):
                    count[0] = min(count[0] + 1, total)
                    on_progress(ProgressStep(count[0], total))

            def chunk(c):
                on_chunk(AudioChunk(c.sample_rate, c.channels, c.samples, index[0]))
                index[0] += 1

            for t in hist.turns:
                track = session.step(t, chunk, progress, decode_now=False)
                if t.role == "assistant" and t.audio is None:
                    parts.append(track)
            on_progress(ProgressDecoding())
            samples: list[float] = []
            for frames in parts:
                samples += session.render(frames, chunk)
            if not samples:
                raise InferenceError(f"{MODEL_ID}: conversation produced no assistant audio")
            return AudioTrack(SAMPLE_RATE, 1, samples)
        chunker = StreamingChunker(self.codec(), frames_per_block(frame_budget(req)), on_chunk)
        self.rvq_frames(req, on_progress, lambda f: chunker.push(f, req.cancel.is_cancelled))
        on_progress(ProgressDecoding())
        pcm = chunker.finish(req.cancel.is_cancelled)
        if pcm is None:
            raise Canceled(f"{MODEL_ID}: cancelled while decoding")
        return AudioTrack(SAMPLE_RATE, 1, pcm.tolist())

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        return GenerationOutput(audio=self._synthesize(req, on_progress, lambda c: None))

    def generate_streaming(self, req: GenerationRequest, on_progress=lambda p: None, on_chunk=lambda c: None) -> GenerationOutput:
        return GenerationOutput(audio=self._synthesize(req, on_progress, on_chunk))

    def open_conversation(self, req: GenerationRequest | None = None) -> "MossConversationSession":
        req = req if req is not None else GenerationRequest()
        self._descriptor.capabilities.validate_request_audio(self._descriptor.id, req)
        decoder, tokenizer = self.pipeline()
        return MossConversationSession(self, decoder, tokenizer, self.reference_codes(req),
                                       req.seed if req.seed is not None else DEFAULT_SAMPLING_SEED, frame_budget(req), req.cancel)


class MossConversationSession(ConversationSession):
    """The conversation's backbone cache stays live across turns: a user turn or an assistant turn with given audio
    only advances it, an assistant turn without audio is synthesised (seeded by the base seed and the count of
    synthesised turns so far) and returned as that turn's track."""

    def __init__(self, gen: MossTtsRealtimeGenerator, decoder: Decoder, tokenizer, reference, base_seed: int, budget: int, cancel):
        self.gen, self.decoder, self.tokenizer, self.reference = gen, decoder, tokenizer, reference
        self.base_seed, self.budget, self.cancel = base_seed, budget, cancel
        self.state, self.turn_index = ConvState(decoder), 0

    def render(self, frames: list[list[int]], on_chunk=lambda c: None) -> list[float]:
        if not frames:
            return []
        codec = self.gen.codec()
        pcm = codec.decode_frames(frames, self.cancel.is_cancelled)
        if pcm is None:
            raise Canceled(f"{MODEL_ID}: cancelled while decoding")
        block = DEFAULT_FRAMES_PER_BLOCK * codec.hop
        for k, o in enumerate(range(0, pcm.numel(), block)):
            on_chunk(AudioChunk(SAMPLE_RATE, 1, pcm[o:o + block].tolist(), k))
        return pcm.tolist()

    def step(self, turn: ConversationTurn, on_chunk=lambda c: None, on_progress=lambda p: None, decode_now: bool = True):
        """-> the turn's AudioTrack (with decode_now=False, used by the single-request path: the turn's frames)."""
        if self.cancel.is_cancelled():
            raise Canceled(f"{MODEL_ID}: cancelled")
        if turn.role not in ("user", "assistant"):
            raise InferenceError(f"{MODEL_ID}: unknown conversation role {turn.role!r}")
        synth = turn.role == "assistant" and turn.audio is None
        prepared = self.gen.prepare_turn(turn, self.turn_index)
        self.turn_index += 1
        count = [0]

        def frame_cb(step, frame):
            count[0] = min(count[0] + 1, self.budget)
            on_progress(ProgressStep(count[0], self.budget))

        frames = advance_turn(self.decoder, self.tokenizer, self.reference, self.state, prepared, self.base_seed, self.budget,
                              self.cancel.is_cancelled, frame_cb)
        if frames is None:
            raise Canceled(f"{MODEL_ID}: cancelled")
        if not decode_now:
            return frames
        on_progress(ProgressDecoding())
        if not synth:
            return turn.audio if turn.audio is not None else AudioTrack(SAMPLE_RATE, 1, [])
        return AudioTrack(SAMPLE_RATE, 1, self.render(frames, on_chunk))


def registration(backend: str) -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> MossTtsRealtimeGenerator:
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
        if src.is_file:
            raise Unsupported(f"{mid} codec component expects a snapshot directory (config.json + model*.safetensors), not the file {src.path}")
        return MossTtsRealtimeGenerator(Path(spec.weights.path), Path(src.path), backend, prefix)

    return Registration(descriptor=lambda: moss_tts_realtime_descriptor(backend, prefix), load=load)


# ---- synthetic checkpoints --------------------------------------------------------------------------------------------------
def random_codec_weights(stages_dec, stages_enc, nq: int, codebook_size: int, codebook_dim: int, rvq_dim: int, code_dim: int,
                         seed: int = 0) -> dict[str, torch.Tensor]:
    """stages_*: (module index, input dim, model dim, output dim, layers, ffn dim) per stage."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)                      # noqa: E731
    w: dict[str, torch.Tensor] = {}

    def wn(p, o, i):
        w[p + ".parametrizations.weight.original1"] = rn(o, i, 1)
        w[p + ".parametrizations.weight.original0"] = (1.0 + 0.1 * rn(o, 1, 1)) * 0.9
        w[p + ".bias"] = rn(o) * 0.02

    wn("quantizer.input_proj", rvq_dim, code_dim)
    wn("quantizer.output_proj", code_dim, rvq_dim)
    for i in range(nq):
        w[f"quantizer.quantizers.{i}.codebook.weight"] = rn(codebook_size, codebook_dim)
        wn(f"quantizer.quantizers.{i}.in_proj", codebook_dim, rvq_dim)
        wn(f"quantizer.quantizers.{i}.out_proj", rvq_dim, codebook_dim)
    for module, stages in (("decoder", stages_dec), ("encoder", stages_enc)):
        for idx, din, d, dout, layers, ffn in stages:
            p = f"{module}.{idx}."
            if din != d:
                w[p + "input_proj.weight"] = rn(d, din) / math.sqrt(din)
            if dout != d:
                w[p + "output_proj.weight"] = rn(dout, d) / math.sqrt(d)
            for li in range(layers):
                b = f"{p}transformer.layers.{li}."
                for n in ("norm1", "norm2"):
                    w[b + n + ".weight"], w[b + n + ".bias"] = 1 + rn(d) * 0.05, rn(d) * 0.02
                w[b + "self_attn.in_projs.0.weight"] = rn(3 * d, d) / math.sqrt(d)
                w[b + "self_attn.out_projs.0.weight"] = rn(d, d) / math.sqrt(d)
                w[b + "linear1.weight"] = rn(ffn, d) / math.sqrt(d)
                w[b + "linear2.weight"] = rn(d, ffn) / math.sqrt(ffn)
                w[b + "layer_scale_1.scale"], w[b + "layer_scale_2.scale"] = 0.3 + 0.05 * rn(d), 0.3 + 0.05 * rn(d)
    return w


SYNTH_CODEC = {"architectures": ["MossAudioTokenizerModel"], "sample_rate": 24_000, "downsample_rate": 24,
               "decoder_patch_sizes": [2, 2, 2, 3], "encoder_patch_sizes": [3, 2, 2, 2], "causal_transformer_context_duration": 0.004,
               "quantizer_kwargs": {"quantizer_type": "rlfq", "num_quantizers": 6, "codebook_size": 8, "codebook_dim": 4,
                                    "rvq_dim": 16, "output_dim": 24}}


def write_synthetic_codec(root, seed: int = 0) -> Path:
    """A tiny codec of the same construction: hop 24 (patches 2 * 2 * 2 * 3), 128-wide stages with two 64-wide heads, and
    a context short enough (4 ms) that the attention band cuts in within a few frames."""
    from ..io.safetensors_io import save_file

    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    (root / "config.json").write_text(json.dumps(SYNTH_CODEC))
    dec = [(0, 24, 128, 128, 2, 64), (2, 64, 128, 128, 1, 64), (4, 64, 128, 128, 1, 64), (6, 64, 128, 3, 1, 64)]
    enc = [(1, 3, 128, 64, 1, 64), (3, 128, 128, 64, 1, 64), (5, 128, 128, 64, 1, 64), (7, 128, 128, 24, 2, 64)]
    q = SYNTH_CODEC["quantizer_kwargs"]
    save_file(random_codec_weights(dec, enc, q["num_quantizers"], q["codebook_size"], q["codebook_dim"], q["rvq_dim"], q["output_dim"],
                                   seed), root / "model.safetensors")
    return root


def write_synthetic_snapshot(root, seed: int = 0) -> tuple[Path, Path]:
    """(model snapshot, codec directory): a 2-layer backbone and depth transformer over 4 codebooks of 8 codes, with a toy
    byte-level tokenizer that knows the markup tokens."""
    import tokenizers
    from tokenizers import decoders, models, pre_tokenizers, trainers

    from ..io.safetensors_io import save_file
    from ..models.oracle import random_llama_weights

    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    specials = ["<|im_start|>", "<|im_end|>", AUDIO_PAD_STR, TEXT_PAD_STR]
    tok = tokenizers.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(["hello there how are you", "fine thanks and you", TTS_SYSTEM_PROMPT, VOICE_CLONE_PREFIX],
                            trainers.BpeTrainer(vocab_size=340, special_tokens=specials, initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tok.save(str(root / "tokenizer.json"))
    vocab, rvq, codes, H = tok.get_vocab_size(), 4, 8, 32
    block = {"hidden_size": H, "intermediate_size": 64, "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1,
             "head_dim": 16, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "attention_bias": False}
    cfg = {"architectures": ["MossTTSRealtime"], "rvq": rvq, "audio_vocab_size": codes + 3, "audio_pad_token": codes,
           "text_pad": tok.token_to_id(TEXT_PAD_STR), "reference_audio_pad": tok.token_to_id(AUDIO_PAD_STR),
           "language_config": {**block, "vocab_size": vocab}, "local_config": {**block, "rvq": rvq, "audio_vocab_size": codes + 3,
                                                                               "audio_pad_token": codes}}
    (root / "config.json").write_text(json.dumps(cfg))
    g = torch.Generator().manual_seed(seed + 1)
    w: dict[str, torch.Tensor] = {}
    lw = random_llama_weights(_llama_config(block, vocab), seed, std=0.3)
    w["embed_tokens.0.weight"] = lw["model.embed_tokens.weight"]
    for k, v in lw.items():
        if k.startswith("model.") and "embed_tokens" not in k:
            w["language_model." + k[len("model."):]] = v
    for c in range(rvq):
        w[f"embed_tokens.{c + 1}.weight"] = torch.randn(codes + 3, H, generator=g) * 0.3
    ll = random_llama_weights(_llama_config(block, codes + 3), seed + 2, std=0.3)
    for k, v in ll.items():
        if k.startswith("model.") and "embed_tokens" not in k:
            w["local_transformer.model." + k[len("model."):]] = v
    for i in range(rvq):
        if i + 1 < rvq:
            w[f"local_transformer.model.embed_tokens.{i}.weight"] = torch.randn(codes + 3, H, generator=g) * 0.3
        w[f"local_transformer.local_lm_heads.{i}.weight"] = torch.randn(codes + 3, H, generator=g) * 0.5
    save_file(w, root / MODEL_WEIGHTS)
    return root, write_synthetic_codec(root.parent / (root.name + "_codec"), seed + 3)
