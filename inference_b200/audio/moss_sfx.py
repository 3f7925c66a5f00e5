"""MOSS-SoundEffect v2 text-to-audio generator `moss_sfx_v2` (parity: candle-audio-moss-sfx/src/{config,text,dit,
sampler,vae,pipeline,model}.rs).

Prompt (+ the trained `" duration: X.Xs"` suffix) -> Qwen3-1.7B hidden states after the final norm, zero-padded to
512 rows -> a Wan-style 1-D DiT over the latent sequence [128 channels, 50 frames per second]: per-block adaLN
(learned table + time projection -> shift / scale / gate), self-attention with model-wide q / k RMSNorm and adjacent-pair
rotary positions, cross-attention to the embedded text (keys / values computed once per prompt), tanh-GELU MLP ->
flow-matching Euler sampler on the shifted sigma schedule -> DAC decoder (Snake activations, transposed-convolution
upsampling x8 x5 x4 x3 x2 = 960 samples per latent frame) -> 48 kHz mono.

The sampler always denoises a whole-second window (the requested length rounded up, at most 30 s) and the track is cut
to the requested length afterwards. Classifier-free guidance runs the negative prompt as a second forward when
guidance != 1.

One implementation for both backends: on a CUDA device the text encoder and every DiT projection / attention call run
on this library's sm_100a kernels in bf16 (nn_dual), the DAC decoder runs in fp32 through the framework's 1-D
convolutions; the CPU backend is the fp32 oracle."""
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
from ..models import nn_dual as nd

MODEL_ID, FAMILY, SAMPLE_RATE, HOP_LENGTH, LATENT_DIM, TEXT_LEN = "moss_sfx_v2", "moss_soundeffect", 48_000, 960, 128, 512
MAX_DURATION_SECS, MAX_SFX_STEPS, GUIDANCE_RANGE, LANGUAGES = 30.0, 1000, (1.0, 20.0), ["en", "zh"]
DEFAULT_SECONDS, DEFAULT_STEPS, DEFAULT_CFG_SCALE = 10.0, 100, 4.0
VAE_FILE = "vae_128d_48k.pth"
DAC_RATES, DAC_DIM = (8, 5, 4, 3, 2), 2048
MOSS_SFX_LICENSE = WeightLicense("Apache-2.0", "Apache License 2.0", "https://huggingface.co/OpenMOSS-Team/MOSS-SoundEffect-v2.0",
                                 "MOSS-SoundEffect v2.0 (c) OpenMOSS Team - licensed under Apache-2.0", True)


# ---- prompt text ----------------------------------------------------------------------------------------------------------
def round_seconds(seconds: float) -> float:
    return math.floor(seconds * 10.0 + 0.5) / 10.0


def with_duration_suffix(prompt: str, seconds: float) -> str:
    return f"{prompt.strip()} duration: {seconds:.1f}s"


def clean_prompt(text: str) -> str:
    """HTML entities unescaped twice (the training pipeline's cleaner), whitespace runs collapsed."""
    return " ".join(_unescape(_unescape(text)).split())


_NAMED = {"amp": "&", "lt": "<", "gt": ">", "quot": '"', "apos": "'", "nbsp": " "}


def _unescape(text: str) -> str:
    out, i = [], 0
    while i < len(text):
        if text[i] == "&":
            semi = text.find(";", i)
            if semi > 0:
                ent, rep = text[i + 1:semi], None
                if ent in _NAMED:
                    rep = _NAMED[ent]
                elif ent.startswith("#"):
                    num = ent[1:]
                    try:
                        cp = int(num[1:], 16) if num[:1] in ("x", "X") else int(num) if num.isdigit() else -1
                        rep = chr(cp) if 0 <= cp < 0x110000 and not 0xD800 <= cp < 0xE000 else None
                    except ValueError:
                        rep = None
                if rep is not None:
                    out.append(rep)
                    i = semi + 1
                    continue
        out.append(text[i])
        i += 1
    return "".join(out)


# ---- schedule -------------------------------------------------------------------------------------------------------------
@dataclass
class SchedulerConfig:
    shift: float = 5.0
    sigma_min: float = 0.0
    extra_one_step: bool = False
    num_train_timesteps: int = 1000


def flow_sigmas(cfg: SchedulerConfig, steps: int, shift: float | None = None) -> list[float]:
    """steps + 1 sigmas from 1 to the terminal 0: `steps` points linear in s from 1 towards sigma_min (spacing 1 / steps
    when `extra_one_step`, else 1 / (steps - 1)), shifted by sigma = shift * s / (1 + (shift - 1) * s), then 0."""
    steps = max(steps, 1)
    sh = cfg.shift if shift is None else shift
    denom = float(steps) if cfg.extra_one_step else max(steps - 1.0, 1.0)
    lin = [1.0 + (cfg.sigma_min - 1.0) * k / denom for k in range(steps)]
    return [sh * s / (1.0 + (sh - 1.0) * s) for s in lin] + [0.0]


# ---- DiT ------------------------------------------------------------------------------------------------------------------
@dataclass
class DitConfig:
    in_dim: int = 128
    out_dim: int = 128
    text_dim: int = 2048
    freq_dim: int = 256
    eps: float = 1e-6
    patch_size: tuple = (1,)
    dim: int = 1536
    ffn_dim: int = 8960
    num_heads: int = 12
    num_layers: int = 30
    has_image_input: bool = False
    vae_type: str = "dac"

    @staticmethod
    def from_json(j: dict) -> "DitConfig":
        c = DitConfig(**{k: j[k] for k in DitConfig.__dataclass_fields__ if k in j})
        c.patch_size = tuple(c.patch_size)
        if c.has_image_input:
            raise LoadError("moss-sfx DiT: has_image_input=true is not the audio checkpoint shape")
        if c.vae_type != "dac":
            raise LoadError(f"moss-sfx DiT: vae_type {c.vae_type!r} unsupported (only the \"dac\" rotary path exists)")
        if c.patch_size != (1,):
            raise LoadError(f"moss-sfx DiT: patch_size {list(c.patch_size)} unsupported (the v2.0 checkpoint uses [1])")
        if c.dim % c.num_heads or (c.dim // c.num_heads) % 2:
            raise LoadError(f"moss-sfx DiT: dim {c.dim} not an even-head multiple of num_heads {c.num_heads}")
        return c


def rope_tables(head_dim: int, length: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(length, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


class SfxDiT:
    def __init__(self, cfg: DitConfig, weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.w = nd.WeightBag(weights, self.dtype, self.device)
        self.heads, self.hd = cfg.num_heads, cfg.dim // cfg.num_heads

    def _mod(self, x, shift, scale):
        return (nd.layer_norm(x, eps=self.cfg.eps).float() * (1.0 + scale.float()) + shift.float()).to(x.dtype)

    def embed_context(self, context: torch.Tensor) -> list[tuple[torch.Tensor, torch.Tensor]]:
        """[1, L, text_dim] -> per block (k, v) [1, L, heads, head_dim] of the embedded text."""
        w, ce = self.w, "condition_embedder.text_embedder."
        ctx = w.lin(w.lin(context.to(self.dtype), ce + "linear_1", act="gelu_tanh"), ce + "linear_2")
        out = []
        for i in range(self.cfg.num_layers):
            p = f"blocks.{i}.attn2."
            k = nd.rms_norm(w.lin(ctx, p + "to_k"), w[p + "norm_k.weight"], self.cfg.eps)
            v = w.lin(ctx, p + "to_v")
            L = ctx.shape[1]
            out.append((k.view(1, L, self.heads, self.hd), v.view(1, L, self.heads, self.hd)))
        return out

    @torch.no_grad()
    def forward(self, latents: torch.Tensor, timestep: float, ctx, cos, sin, cancel=lambda: False) -> torch.Tensor | None:
        """latents [1, in_dim, T] at `timestep` (sigma * 1000) -> velocity [1, out_dim, T]; None when cancelled."""
        cfg, w, H, D = self.cfg, self.w, self.heads, self.hd
        t_emb = nd.sinusoidal_embedding(torch.tensor([timestep], device=self.device), cfg.freq_dim).to(self.dtype)
        ce = "condition_embedder."
        t = w.lin(w.lin(t_emb, ce + "time_embedder.linear_1", act="silu"), ce + "time_embedder.linear_2")      # [1, dim]
        t_mod = w.lin(F.silu(t.float()).to(self.dtype), ce + "time_proj").view(1, 6, cfg.dim)
        pw = w["patch_embedding.weight"]                     # [dim, in_dim, 1]: patch 1 makes the convolution a projection
        x = nd.linear(latents.to(self.dtype).transpose(1, 2), pw.reshape(pw.shape[0], -1), w["patch_embedding.bias"])
        T = x.shape[1]
        for i in range(cfg.num_layers):
            if cancel():
                return None
            p = f"blocks.{i}."
            m = (w[p + "scale_shift_table"].float() + t_mod.float())
            sm, cm, gm, sf, cf, gf = (m[:, j:j + 1] for j in range(6))
            h = self._mod(x, sm, cm)
            a = p + "attn1."
            q = nd.rms_norm(w.lin(h, a + "to_q"), w[a + "norm_q.weight"], cfg.eps).view(1, T, H, D)
            k = nd.rms_norm(w.lin(h, a + "to_k"), w[a + "norm_k.weight"], cfg.eps).view(1, T, H, D)
            v = w.lin(h, a + "to_v").view(1, T, H, D)
            o = nd.attention(nd.rope_interleaved(q, cos, sin), nd.rope_interleaved(k, cos, sin), v)
            x = (x.float() + w.lin(o, a + "to_out.0").float() * gm).to(self.dtype)
            c = p + "attn2."
            hq = nd.layer_norm(x, w[p + "norm2.weight"], w[p + "norm2.bias"], cfg.eps)
            q = nd.rms_norm(w.lin(hq, c + "to_q"), w[c + "norm_q.weight"], cfg.eps).view(1, T, H, D)
            ck, cv = ctx[i]
            x = x + w.lin(nd.attention(q, ck, cv), c + "to_out.0")
            h = self._mod(x, sf, cf)
            f = w.lin(w.lin(h, p + "ffn.net.0.proj", act="gelu_tanh"), p + "ffn.net.2")
            x = (x.float() + f.float() * gf).to(self.dtype)
        m = w["scale_shift_table"].float() + t.float()[:, None]
        x = self._mod(x, m[:, 0:1], m[:, 1:2])
        return w.lin(x, "proj_out").float().transpose(1, 2).contiguous()


# ---- DAC decoder ----------------------------------------------------------------------------------------------------------
def fold_weight_norm(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """`weight_g` / `weight_v` pairs -> `weight` = g * v / ||v|| (norm over every axis but the first)."""
    out = {}
    for k, v in sd.items():
        if k.endswith(".weight_g"):
            base = k[: -len("weight_g")]
            wv = sd[base + "weight_v"].float()
            n = wv.flatten(1).norm(dim=1).view(-1, *([1] * (wv.dim() - 1)))
            out[base + "weight"] = v.float() * wv / n
        elif not k.endswith(".weight_v"):
            out[k] = v.float() if v.is_floating_point() else v
    return out


def snake(x: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """x + sin^2(alpha x) / (alpha + 1e-9), alpha per channel [1, C, 1]."""
    return x + torch.sin(alpha * x).pow(2) / (alpha + 1e-9)


class DacDecoder:
    """Latent [1, 128, T] -> waveform [1, 1, T * 960]: a 1x1 `post_quant_conv`, a width-7 stem, one block per upsampling
    rate (Snake, transposed convolution of kernel 2 * rate, three residual units with dilations 1 / 3 / 9), Snake, a
    width-7 head and tanh. Channel width halves per block from 2048."""

    def __init__(self, weights: dict[str, torch.Tensor], device="cpu", rates=DAC_RATES):
        self.device, self.rates = torch.device(device), tuple(rates)
        self.w = {k: v.to(self.device) for k, v in fold_weight_norm(weights).items()}

    def _conv(self, x, p, **kw):
        return F.conv1d(x, self.w[p + ".weight"], self.w.get(p + ".bias"), **kw)

    @torch.no_grad()
    def decode(self, z: torch.Tensor, cancel=lambda: False) -> torch.Tensor | None:
        w = self.w
        x = self._conv(z.float().to(self.device), "post_quant_conv")
        x = self._conv(x, "decoder.model.0", padding=3)
        for i, r in enumerate(self.rates):
            if cancel():
                return None
            p = f"decoder.model.{i + 1}.block."
            x = snake(x, w[p + "0.alpha"])
            x = F.conv_transpose1d(x, w[p + "1.weight"], w.get(p + "1.bias"), stride=r, padding=math.ceil(r / 2), output_padding=r % 2)
            for j, dil in enumerate((1, 3, 9)):
                u = f"{p}{j + 2}.block."
                y = self._conv(snake(x, w[u + "0.alpha"]), u + "1", padding=3 * dil, dilation=dil)
                x = x + self._conv(snake(y, w[u + "2.alpha"]), u + "3")
        n = len(self.rates) + 1
        x = snake(x, w[f"decoder.model.{n}.alpha"])
        return torch.tanh(self._conv(x, f"decoder.model.{n + 1}", padding=3))


def load_dac_weights(vae_dir: Path) -> dict[str, torch.Tensor]:
    pth, st = vae_dir / VAE_FILE, vae_dir / (VAE_FILE[:-4] + ".safetensors")
    if st.is_file():
        from ..io.safetensors_io import load_file

        return load_file(st)
    if not pth.is_file():
        raise LoadError(f"moss-sfx: {pth} missing")
    sd = torch.load(pth, map_location="cpu", weights_only=True)
    sd = sd.get("state_dict", sd)
    return {k: v for k, v in sd.items() if k.startswith(("decoder.", "post_quant_conv."))}


# ---- pipeline -------------------------------------------------------------------------------------------------------------
class MossSfxPipeline:
    def __init__(self, root: Path, device="cpu"):
        from ..io.safetensors_io import load_dir, load_file
        from ..contracts.gen_core.tokenizer import TextTokenizer, TokenizerConfig
        from ..models.config import ModelConfig
        from ..models.text_encoders import CausalLmTextEncoder

        root = Path(root)

        def read(rel):
            f = root / rel
            if not f.is_file():
                raise LoadError(f"moss-sfx snapshot {root} has no {rel}")
            return json.loads(f.read_text(encoding="utf-8"))

        idx = read("model_index.json")
        if idx.get("_class_name") != "MossSoundEffectPipeline":
            raise LoadError(f"{root} is not a MOSS-SoundEffect snapshot (_class_name {idx.get('_class_name')!r})")
        if idx.get("vae_type", "dac") != "dac":
            raise LoadError(f"moss-sfx: vae_type {idx['vae_type']!r} unsupported (only \"dac\")")
        self.sample_rate = int(idx.get("sample_rate", SAMPLE_RATE))
        self.max_seconds = int(idx.get("max_inference_seconds", 30))
        sj = read("scheduler/scheduler_config.json")
        self.scheduler = SchedulerConfig(**{k: sj[k] for k in SchedulerConfig.__dataclass_fields__ if k in sj})
        self.dit_cfg = DitConfig.from_json(read("transformer/config.json"))
        tj = read("text_encoder/config.json")
        if tj.get("use_sliding_window"):
            raise LoadError("moss-sfx text encoder: sliding-window attention is not implemented (the pinned config has it off)")
        if tj["hidden_size"] != self.dit_cfg.text_dim:
            raise LoadError(f"moss-sfx: text encoder hidden_size {tj['hidden_size']} != DiT text_dim {self.dit_cfg.text_dim}")
        if self.dit_cfg.in_dim != LATENT_DIM:
            raise LoadError(f"moss-sfx: DiT in_dim {self.dit_cfg.in_dim} != VAE latent dim {LATENT_DIM}")
        self.device = torch.device(device)
        tk = root / "tokenizer" / "tokenizer.json"
        if not tk.is_file():
            raise LoadError(f"moss-sfx snapshot {root} has no tokenizer/tokenizer.json")
        self.tokenizer = TextTokenizer.from_file(tk, TokenizerConfig(max_length=TEXT_LEN))
        tcfg = ModelConfig.from_json({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", **tj})
        self.text = CausalLmTextEncoder(tcfg, load_dir(root / "text_encoder"), self.device, skip_last=0, final_norm=True)
        self.dit = SfxDiT(self.dit_cfg, load_file(root / "transformer" / "diffusion_pytorch_model.safetensors"), self.device)
        self.vae = DacDecoder(load_dac_weights(root / "vae"), self.device, idx.get("dac_rates", DAC_RATES))
        self.hop = math.prod(self.vae.rates)

    def encode_context(self, prompt: str) -> torch.Tensor:
        cleaned = clean_prompt(prompt)
        ids = self.tokenizer.encode_ids(cleaned, True)[:TEXT_LEN] if cleaned else []
        D = self.dit_cfg.text_dim
        if not ids:
            return torch.zeros(1, TEXT_LEN, D, device=self.device)
        h = self.text.encode(ids).float()
        return F.pad(h, (0, 0, 0, TEXT_LEN - h.shape[1]))

    def window_seconds(self, seconds: float) -> int:
        return min(max(int(math.ceil(seconds)), 1), self.max_seconds)

    @torch.no_grad()
    def synthesize(self, prompt: str, seconds: float, steps: int, cfg_scale: float, negative: str, seed: int,
                   sigma_shift: float | None = None, on_step=lambda k: None, on_decode=lambda: None,
                   cancel=lambda: False) -> torch.Tensor:
        from ..media.seed import seeded_normal

        seconds = round_seconds(seconds)
        if seconds <= 0:
            raise InferenceError(f"moss-sfx: seconds must be > 0 after 0.1 s rounding (got {seconds})")
        T = self.window_seconds(seconds) * self.sample_rate // self.hop
        ctx_pos = self.dit.embed_context(self.encode_context(with_duration_suffix(prompt, seconds)))
        ctx_neg = self.dit.embed_context(self.encode_context(negative)) if cfg_scale != 1.0 else None
        sig = flow_sigmas(self.scheduler, steps, sigma_shift)
        cos, sin = rope_tables(self.dit.hd, T, self.device)
        x = seeded_normal(seed, self.dit_cfg.in_dim * T).view(1, self.dit_cfg.in_dim, T).to(self.device)
        for k in range(steps):
            t = sig[k] * self.scheduler.num_train_timesteps
            v = self.dit.forward(x, t, ctx_pos, cos, sin, cancel)
            if v is not None and ctx_neg is not None:
                vn = self.dit.forward(x, t, ctx_neg, cos, sin, cancel)
                v = None if vn is None else vn + (v - vn) * cfg_scale
            if v is None or cancel():
                raise Canceled(f"{MODEL_ID}: cancelled at step {k}")
            x = x + v * (sig[k + 1] - sig[k])
            on_step(k + 1)
        on_decode()
        audio = self.vae.decode(x, cancel)
        if audio is None:
            raise Canceled(f"{MODEL_ID}: cancelled while decoding")
        full = audio.reshape(-1).float().cpu()
        return full[: min(int(round(self.sample_rate * seconds)), full.numel())]


# ---- generator ------------------------------------------------------------------------------------------------------------
def moss_sfx_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family=FAMILY, backend=backend, modality=Modality.AUDIO,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False, conditioning=[],
            supports_lora=False, supports_lokr=False, samplers=[], schedulers=[], supported_guidance_methods=[],
            min_size=0, max_size=0, max_count=1, audio_sample_rates=[SAMPLE_RATE], max_audio_duration_secs=MAX_DURATION_SECS,
            audio_voices=[], audio_languages=list(LANGUAGES)),
        required_components=[])


class MossSfxGenerator(Generator):
    def __init__(self, root: Path, backend: str, prefix: str = ""):
        self.root, self.backend = Path(root), backend
        self._descriptor = moss_sfx_descriptor(backend, prefix)
        self._pipe: MossSfxPipeline | None = None

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        if not req.prompt.strip():
            raise InferenceError(f"{mid}: prompt (the sound description) must not be empty")
        self._descriptor.capabilities.validate_request_audio(mid, req)
        if req.steps is not None and req.steps > MAX_SFX_STEPS:
            raise InferenceError(f"{mid}: steps {req.steps} exceeds the schedule's {MAX_SFX_STEPS} training timesteps")
        if req.guidance is not None and not (GUIDANCE_RANGE[0] <= req.guidance <= GUIDANCE_RANGE[1]):
            raise InferenceError(f"{mid}: guidance {req.guidance} outside {GUIDANCE_RANGE[0]}..={GUIDANCE_RANGE[1]}")
        if req.scheduler_shift is not None and not (math.isfinite(req.scheduler_shift) and req.scheduler_shift > 0):
            raise InferenceError(f"{mid}: scheduler_shift must be a positive finite number")
        a = req.audio
        if a is not None and a.target_duration is not None and round_seconds(a.target_duration) <= 0:
            raise InferenceError(f"{mid}: audio.target_duration rounds to 0.0 s on the model's 0.1 s grid")

    def pipeline(self) -> MossSfxPipeline:
        if self._pipe is None:
            self._pipe = MossSfxPipeline(self.root, "cuda" if self.backend == "b200" else "cpu")
        return self._pipe

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        self.validate(req)
        if req.cancel.is_cancelled():
            raise Canceled(f"{self._descriptor.id}: cancelled")
        from ..media.seed import default_seed

        a = req.audio
        steps = req.steps if req.steps is not None else DEFAULT_STEPS
        samples = self.pipeline().synthesize(
            req.prompt, a.target_duration if a is not None and a.target_duration is not None else DEFAULT_SECONDS, steps,
            req.guidance if req.guidance is not None else DEFAULT_CFG_SCALE, req.negative_prompt or "",
            req.seed if req.seed is not None else default_seed(), req.scheduler_shift,
            on_step=lambda k: on_progress(ProgressStep(k, steps)), on_decode=lambda: on_progress(ProgressDecoding()),
            cancel=req.cancel.is_cancelled)
        return GenerationOutput(audio=AudioTrack(SAMPLE_RATE, 1, samples.tolist()))


def registration(backend: str) -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> MossSfxGenerator:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise LoadError(f"{mid} expects a snapshot directory (model_index.json + text_encoder/ + transformer/ + vae/)")
        if spec.quantize is not None:
            raise Unsupported(f"{mid} does not support on-the-fly quantization")
        if spec.adapters:
            raise Unsupported(f"{mid} does not support LoRA/LoKr adapters")
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid} does not support control/IP-adapter overlays")
        return MossSfxGenerator(Path(spec.weights.path), backend, prefix)

    return Registration(descriptor=lambda: moss_sfx_descriptor(backend, prefix), load=load)


# ---- synthetic snapshot -----------------------------------------------------------------------------------------------------
def random_dit_weights(cfg: DitConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    w["patch_embedding.weight"], w["patch_embedding.bias"] = rn(cfg.dim, cfg.in_dim, 1) * 0.1, rn(cfg.dim) * 0.02
    ce = "condition_embedder."
    lin(w, ce + "text_embedder.linear_1", cfg.dim, cfg.text_dim)
    lin(w, ce + "text_embedder.linear_2", cfg.dim, cfg.dim)
    lin(w, ce + "time_embedder.linear_1", cfg.dim, cfg.freq_dim)
    lin(w, ce + "time_embedder.linear_2", cfg.dim, cfg.dim)
    lin(w, ce + "time_proj", 6 * cfg.dim, cfg.dim)
    for i in range(cfg.num_layers):
        p = f"blocks.{i}."
        for a in ("attn1.", "attn2."):
            for n in ("to_q", "to_k", "to_v", "to_out.0"):
                lin(w, p + a + n, cfg.dim, cfg.dim)
            w[p + a + "norm_q.weight"], w[p + a + "norm_k.weight"] = 1 + rn(cfg.dim) * 0.05, 1 + rn(cfg.dim) * 0.05
        w[p + "norm2.weight"], w[p + "norm2.bias"] = 1 + rn(cfg.dim) * 0.05, rn(cfg.dim) * 0.02
        lin(w, p + "ffn.net.0.proj", cfg.ffn_dim, cfg.dim)
        lin(w, p + "ffn.net.2", cfg.dim, cfg.ffn_dim)
        w[p + "scale_shift_table"] = rn(1, 6, cfg.dim) * 0.1
    w["scale_shift_table"] = rn(1, 2, cfg.dim) * 0.1
    lin(w, "proj_out", cfg.out_dim, cfg.dim)
    return w


def random_dac_weights(dim: int, rates=DAC_RATES, latent: int = LATENT_DIM, seed: int = 0) -> dict[str, torch.Tensor]:
    """Old-style weight-norm layout (`weight_g` / `weight_v`), as the checkpoint stores it."""
    g = torch.Generator().manual_seed(seed)
    w: dict[str, torch.Tensor] = {}

    def conv(p, o, i, k, transposed=False):
        shape = (i, o, k) if transposed else (o, i, k)
        w[p + ".weight_v"] = torch.randn(*shape, generator=g) * (1.0 / math.sqrt(i * k))
        w[p + ".weight_g"] = w[p + ".weight_v"].flatten(1).norm(dim=1).view(-1, 1, 1) * (0.8 + 0.4 * torch.rand(shape[0], 1, 1, generator=g))
        w[p + ".bias"] = torch.randn(o, generator=g) * 0.01

    w["post_quant_conv.weight"], w["post_quant_conv.bias"] = torch.randn(latent, latent, 1, generator=g) * 0.1, torch.zeros(latent)
    conv("decoder.model.0", dim, latent, 7)
    c = dim
    for i, r in enumerate(rates):
        p = f"decoder.model.{i + 1}.block."
        w[p + "0.alpha"] = torch.rand(1, c, 1, generator=g) + 0.5
        conv(p + "1", c // 2, c, 2 * r, transposed=True)
        c //= 2
        for j in range(3):
            u = f"{p}{j + 2}.block."
            w[u + "0.alpha"], w[u + "2.alpha"] = torch.rand(1, c, 1, generator=g) + 0.5, torch.rand(1, c, 1, generator=g) + 0.5
            conv(u + "1", c, c, 7)
            conv(u + "3", c, c, 1)
    n = len(rates) + 1
    w[f"decoder.model.{n}.alpha"] = torch.rand(1, c, 1, generator=g) + 0.5
    conv(f"decoder.model.{n + 1}", 1, c, 7)
    return w


def write_synthetic_snapshot(root, seed: int = 0, sample_rate: int = SAMPLE_RATE) -> Path:
    """A tiny random MOSS-SoundEffect-shaped snapshot: 2-block DiT of width 32, a 3-layer Qwen3 text encoder with a toy
    byte-level tokenizer, a 64-wide DAC decoder with the real upsampling rates."""
    from ..io.safetensors_io import save_file
    from ..media.z_image import _write_synthetic_qwen3

    root = Path(root)
    for d in ("scheduler", "transformer", "vae"):
        (root / d).mkdir(parents=True, exist_ok=True)
    (root / "model_index.json").write_text(json.dumps({"_class_name": "MossSoundEffectPipeline", "sample_rate": sample_rate,
                                                       "max_inference_seconds": 30, "vae_type": "dac"}))
    (root / "scheduler" / "scheduler_config.json").write_text(json.dumps({"shift": 5.0, "sigma_min": 0.0, "extra_one_step": True,
                                                                          "num_train_timesteps": 1000}))
    cfg = DitConfig(text_dim=24, freq_dim=16, dim=32, ffn_dim=64, num_heads=2, num_layers=2)
    (root / "transformer" / "config.json").write_text(json.dumps({**cfg.__dict__, "patch_size": [1]}))
    save_file(random_dit_weights(cfg, seed), root / "transformer" / "diffusion_pytorch_model.safetensors")
    _write_synthetic_qwen3(root, 24, 12, seed + 1)
    save_file(random_dac_weights(64, seed=seed + 2), root / "vae" / (VAE_FILE[:-4] + ".safetensors"))
    return root
