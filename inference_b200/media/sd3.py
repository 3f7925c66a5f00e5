"""Stable Diffusion 3.5 providers `sd3_5_large`, `sd3_5_large_turbo`, `sd3_5_medium` (and `cpu_*` on the fp32 backend)
(parity: candle-gen-sd3/src/lib.rs, pipeline.rs, conditioning.rs, vae.rs).

Conditioning: CLIP-L and CLIP-G second-to-last hidden states concatenated on the feature axis ([77, 2048], zero-padded
to the T5 width) followed by T5 ([256, 4096], padding attended) -> context [333, 4096]; pooled = the two projected CLIP
vectors concatenated [2048]. Sampling: flow-match Euler over the shift-3 table, the model's timestep is sigma * 1000,
classifier-free guidance `uncond + g * (cond - uncond)` (Large 28 steps / 4.0, Medium 40 / 4.5); Large Turbo is
guidance-distilled (4 steps, no negative prompt). The VAE is the 16-channel autoencoder with scaling 1.5305 and shift
0.0609.

Snapshot layout (diffusers): `transformer/`, `text_encoder/` + `tokenizer/` (CLIP-L), `text_encoder_2/` + `tokenizer_2/`
(CLIP-G), `text_encoder_3/` + `tokenizer_3/` (T5), `vae/`; `swb_config.json` overrides dimensions for synthetic
snapshots."""
from __future__ import annotations

import enum
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, GenerationOutput, GenerationRequest, Generator,
                                            Modality, ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import AdapterKind, LoadSpec, OffloadPolicy, ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import (SCHEDULERS, SOLVERS, FlowModelSampling, TorchLatentOps, denoise, get_solver,
                                           schedule_sigmas)
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.dit_sd3 import Sd3Config, Sd3DiT
from ..models.vae import OracleVaeDecoder, VaeConfig
from .chroma import convert_diffusers_vae_decoder, native_vae_to_diffusers
from .flux import SIZE_MULTIPLE
from .residency import Residency
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw

SCHEDULE_SHIFT = 3.0
T5_TOKENS = 256
VAE_SCALE, VAE_SHIFT = 1.5305, 0.0609


def sd3_sigmas(steps: int, shift: float = SCHEDULE_SHIFT) -> list[float]:
    """`steps` values evenly spaced from 1 to 1 / 1000, each through the static shift `s x / (1 + (s - 1) x)`, then 0
    (candle-gen-sd3/src/pipeline.rs:118-138; four steps at shift 3 give 1, 0.8573, 0.6007, 0.002994, 0)."""
    n = max(1, steps)
    ramp = [1.0 - (0.0 if n == 1 else i / (n - 1)) * (1.0 - 1.0 / 1000.0) for i in range(n)]
    return [shift * s / (1.0 + (shift - 1.0) * s) for s in ramp] + [0.0]


class Sd3Variant(enum.Enum):
    LARGE = "sd3_5_large"
    LARGE_TURBO = "sd3_5_large_turbo"
    MEDIUM = "sd3_5_medium"

    @property
    def default_steps(self) -> int:
        return {Sd3Variant.LARGE: 28, Sd3Variant.LARGE_TURBO: 4, Sd3Variant.MEDIUM: 40}[self]

    @property
    def default_guidance(self) -> float:
        return {Sd3Variant.LARGE: 4.0, Sd3Variant.LARGE_TURBO: 1.0, Sd3Variant.MEDIUM: 4.5}[self]

    @property
    def uses_cfg(self) -> bool:
        return self is not Sd3Variant.LARGE_TURBO

    def dit_config(self) -> Sd3Config:
        return Sd3Config.medium() if self is Sd3Variant.MEDIUM else Sd3Config.large()


@dataclass
class Sd3Conditioning:
    context: torch.Tensor        # [1, 77 + T5 tokens, joint_attention_dim]
    pooled: torch.Tensor         # [1, pooled_projection_dim]


class TripleTextEncoders:
    def __init__(self, clip_l, tok_l, clip_g, tok_g, t5, tok_t5, width: int, t5_tokens: int = T5_TOKENS):
        self.clip_l, self.tok_l, self.clip_g, self.tok_g = clip_l, tok_l, clip_g, tok_g
        self.t5, self.tok_t5, self.width, self.t5_tokens = t5, tok_t5, width, t5_tokens

    @staticmethod
    def from_snapshot(root: Path, backend: str, device, width: int) -> "TripleTextEncoders":
        from ..models.text_encoders import ClipTextConfig, ClipTextEncoder, T5Config, T5Encoder
        from .text_models import ClipBpeTokenizer, T5SentencePieceTokenizer, _load_component

        dtype = torch.bfloat16 if backend == "b200" else torch.float32
        need = ["text_encoder", "text_encoder_2", "text_encoder_3", "tokenizer", "tokenizer_2", "tokenizer_3"]
        missing = [d for d in need if not (root / d).is_dir()]
        if missing:
            raise LoadError(f"sd3 snapshot {root}: missing text-encoder components {missing}")
        clips = []
        for enc, tok in (("text_encoder", "tokenizer"), ("text_encoder_2", "tokenizer_2")):
            cj, cw = _load_component(root / enc)
            cfg = ClipTextConfig.from_json(cj)
            clips += [ClipTextEncoder(cfg, cw, device, dtype), ClipBpeTokenizer.from_dir(root / tok, cfg.max_position_embeddings)]
        tj, tw = _load_component(root / "text_encoder_3")
        return TripleTextEncoders(*clips, T5Encoder(T5Config.from_json(tj), tw, device, dtype),
                                  T5SentencePieceTokenizer(root / "tokenizer_3" / "spiece.model"), width)

    def encode(self, prompt: str) -> Sd3Conditioning:
        # CLIP-L pads with its end token, CLIP-G with token 0 (their tokenizer configurations)
        l = self.clip_l.encode_all(torch.tensor([self.tok_l.encode(prompt)], dtype=torch.int64))
        g = self.clip_g.encode_all(torch.tensor([self.tok_g.encode(prompt, pad_id=0)], dtype=torch.int64))
        t5 = self.t5.encode(torch.tensor([self.tok_t5.encode(prompt, self.t5_tokens)], dtype=torch.int64))
        clip = torch.cat([l["penultimate"], g["penultimate"]], -1)
        clip = torch.nn.functional.pad(clip, (0, self.width - clip.shape[-1]))
        pooled = torch.cat([l.get("projected", l["pooled"]), g.get("projected", g["pooled"])], -1)
        return Sd3Conditioning(torch.cat([clip.to(t5.dtype), t5], 1), pooled)


class HashTripleEncoders:
    """Weight-free stand-in (synthetic snapshots)."""

    def __init__(self, width: int, pooled: int, device, dtype):
        from .text_encoders import HashTextEncoders

        self.h = HashTextEncoders(width, pooled, device, dtype)

    def encode(self, prompt: str) -> Sd3Conditioning:
        c = self.h.encode(prompt, 24)
        return Sd3Conditioning(c.txt, c.pooled)


@dataclass
class _Heavy:
    dit: Any
    vae: Any


class Sd3Pipeline:
    def __init__(self, variant: Sd3Variant, root: Path, backend: str, device: torch.device):
        self.variant, self.root, self.backend, self.device = variant, Path(root), backend, device
        self.dit_cfg = variant.dit_config()
        self.vae_cfg = VaeConfig(scale_factor=VAE_SCALE, shift_factor=VAE_SHIFT)
        self.text_kind, self.random_init, self.adapters = "triple", None, []
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            raw = json.loads(cfg_path.read_text())
            if "dit" in raw:
                self.dit_cfg = Sd3Config.from_json(raw["dit"])
            if "vae" in raw:
                v = dict(raw["vae"])
                if "ch_mult" in v:
                    v["ch_mult"] = tuple(v["ch_mult"])
                self.vae_cfg = VaeConfig(**{"scale_factor": VAE_SCALE, "shift_factor": VAE_SHIFT, **v})
            self.text_kind = raw.get("text", self.text_kind)
            self.random_init = raw.get("random_init")
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = Sd3Config.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32

    def load_text(self):
        if self.text_kind == "hash":
            return HashTripleEncoders(self.dit_cfg.joint_attention_dim, self.dit_cfg.pooled_projection_dim, self.device,
                                      self.dtype)
        return TripleTextEncoders.from_snapshot(self.root, self.backend, self.device, self.dit_cfg.joint_attention_dim)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir, load_file
        from ..models.dit_sd3 import random_sd3_weights
        from ..models.vae import random_vae_weights

        gpu = self.backend == "b200"
        if self.random_init is not None and gpu:
            seed = int(self.random_init)
            dit_w = random_sd3_weights(self.dit_cfg, seed, 0.02, torch.bfloat16, self.device)
            vae_w = random_vae_weights(self.vae_cfg, seed + 1, dtype=torch.bfloat16, device=self.device)
        else:
            for d in ("transformer", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{self.variant.value}: snapshot {self.root} lacks {d}/")
            dit_w = load_dir(self.root / "transformer")
            for ad in self.adapters:
                from .train import merge_lora

                if not Path(ad.path).is_file():
                    raise LoadError(f"{self.variant.value}: adapter file {ad.path} not found")
                dit_w = merge_lora(dit_w, load_file(ad.path), ad.scale if ad.scale is not None else 1.0)
            vae_w = convert_diffusers_vae_decoder(load_dir(self.root / "vae"), len(self.vae_cfg.ch_mult))
        dit = Sd3DiT(self.dit_cfg, dit_w, self.dtype, self.device)
        if gpu:
            from ..models.vae import VaeDecoderGpu

            return _Heavy(dit, VaeDecoderGpu(self.vae_cfg, self.device).load_state_dict(vae_w))
        return _Heavy(dit, OracleVaeDecoder(self.vae_cfg, vae_w, device=self.device))

    def guidance(self, req: GenerationRequest) -> float:
        if not self.variant.uses_cfg:
            return 1.0
        return float(req.guidance) if req.guidance is not None else self.variant.default_guidance

    def encode(self, text, req: GenerationRequest):
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt or "") if self.guidance(req) > 1.0 else None
        return pos, neg

    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        v = self.variant
        steps = req.steps or v.default_steps
        guidance = self.guidance(req)
        base_seed = req.seed if req.seed is not None else default_seed()
        lh, lw = req.height // 8, req.width // 8
        dev, dt = self.device, self.dtype
        if req.scheduler is None:
            sigmas = sd3_sigmas(steps)
        else:
            sigmas = schedule_sigmas(req.scheduler, FlowModelSampling(mu=req.scheduler_shift or 0.0), steps)
        solver, ops, ms = get_solver(req.sampler or "euler"), TorchLatentOps(), FlowModelSampling()
        from .chroma import convert_diffusers_vae_encoder
        from .reference import encode_reference_image, init_time_step, reference_of

        ref = reference_of(req, v.value)
        clean, start = None, 0
        if ref is not None and init_time_step(steps, ref[1]) > 0:
            from ..io.safetensors_io import load_dir

            start = min(init_time_step(steps, ref[1]), len(sigmas) - 2)
            clean = encode_reference_image(self.vae_cfg, convert_diffusers_vae_encoder(load_dir(self.root / "vae")), ref[0],
                                           req.width, req.height, dev, v.value).to(dev)
            sigmas = sigmas[start:]                    # the run enters the schedule at sigma_start
        conds = [c for c in cond if c is not None]
        # both guidance branches share every shape: one batched forward per step
        context = torch.cat([c.context for c in conds], 0).to(dev, dt)
        pooled = torch.cat([c.pooled for c in conds], 0).to(dev, dt)
        nb = len(conds)

        def one_image(seed: int) -> Image:
            x = seeded_noise_nchw(seed, self.vae_cfg.z_channels, lh, lw).to(dev)
            if clean is not None:                       # x_t = (1 - sigma) clean + sigma noise at the entry point
                x = (1.0 - sigmas[0]) * clean + sigmas[0] * x.float()
            x = x.to(dt).contiguous()
            state = {"step": start}
            for s_done in range(1, start + 1):
                on_progress(ProgressStep(s_done, steps))

            def run_model(x_in, sigma):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{v.value}: cancelled at step {state['step']}")
                tt = torch.full((nb,), float(sigma) * 1000.0, device=dev)
                o = heavy.dit.forward(x_in.expand(nb, -1, -1, -1), tt, context, pooled).float()
                vel = o[0:1] if nb == 1 else o[1:2] + (o[0:1] - o[1:2]) * guidance
                state["step"] += 1
                if state["step"] <= steps:
                    on_progress(ProgressStep(state["step"], steps))
                return vel.to(dt).contiguous()

            x = solver.sample(ops, ms, lambda xx, s: denoise(ops, ms, xx, s, run_model), x, sigmas, seed)
            while state["step"] < steps:
                state["step"] += 1
                on_progress(ProgressStep(state["step"], steps))
            if req.cancel.is_cancelled():
                raise Canceled(f"{v.value}: cancelled before decode")
            on_progress(ProgressDecoding())
            z = x.float()
            if self.backend == "b200":
                host = heavy.vae.decode_rgb8(z)[0].cpu()
            else:
                img = heavy.vae.decode(z)[0].permute(1, 2, 0)
                host = torch.round((img.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).cpu()
            return Image(width=req.width, height=req.height, pixels=host.contiguous().numpy().tobytes())

        return for_each_image_seed(base_seed, req.count, one_image)


def sd3_descriptor(variant: Sd3Variant, backend: str, prefix: str = "") -> ModelDescriptor:
    cfg = variant.uses_cfg
    return ModelDescriptor(
        id=prefix + variant.value, family="sd3", backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=cfg, supports_guidance=cfg, supports_true_cfg=False,
            conditioning=[ConditioningKind.REFERENCE],
            supports_lora=True, supports_lokr=False, samplers=list(SOLVERS), schedulers=list(SCHEDULERS),
            supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8,
            supports_sequential_offload=True),
        required_components=[])


class Sd3Generator(Generator):
    def __init__(self, pipe: Sd3Pipeline, descriptor: ModelDescriptor, policy: OffloadPolicy):
        self.pipe, self._descriptor = pipe, descriptor
        sync = torch.cuda.synchronize if pipe.backend == "b200" else (lambda: None)
        self.residency = Residency.from_policy(policy, pipe.load_text, pipe.load_heavy, sync)

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        self._descriptor.capabilities.validate_request(mid, req)
        if not req.prompt:
            raise InferenceError(f"{mid}: prompt must not be empty")
        if req.steps == 0:
            raise InferenceError(f"{mid}: steps must be >= 1")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} "
                                 f"(got {req.width}x{req.height})")
        side = self.pipe.dit_cfg.pos_embed_max_size * self.pipe.dit_cfg.patch_size * 8
        if req.width > side or req.height > side:
            raise InferenceError(f"{mid}: the position table covers at most {side}x{side} pixels")

    def generate(self, req: GenerationRequest, on_progress: Callable = lambda p: None) -> GenerationOutput:
        self.validate(req)
        images = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(images=images)


def _load(variant: Sd3Variant, backend: str, prefix: str) -> Callable[[LoadSpec], Sd3Generator]:
    def load(spec: LoadSpec) -> Sd3Generator:
        mid = prefix + variant.value
        if spec.weights is None or spec.weights.is_file:
            raise Unsupported(f"{mid}: needs a snapshot directory")
        if spec.quantize is not None:
            raise Unsupported(f"{mid}: quantised loading ({spec.quantize.name}) is not supported")
        reject_unknown_components(spec.components, [], mid)
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid}: control branches and IP adapters are not supported by this provider")
        for ad in spec.adapters:
            if ad.kind is not AdapterKind.LORA:
                raise Unsupported(f"{mid}: adapter kind {ad.kind.value} is not supported (lora)")
        if backend == "b200":
            if not torch.cuda.is_available():
                raise LoadError(f"{mid}: no CUDA device")
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
        pipe = Sd3Pipeline(variant, Path(spec.weights.path), backend, device)
        pipe.adapters = list(spec.adapters)
        return Sd3Generator(pipe, sd3_descriptor(variant, backend, prefix), spec.offload_policy)
    return load


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=(lambda v=v: sd3_descriptor(v, backend, prefix)), load=_load(v, backend, prefix))
            for v in (Sd3Variant.LARGE, Sd3Variant.LARGE_TURBO, Sd3Variant.MEDIUM)]


def write_synthetic_snapshot(root, seed: int = 0, dual: bool = False) -> Path:
    """A tiny random SD3-shaped snapshot in the diffusers directory layout with the weight-free prompt encoder
    (dual=True gives the first block a second, image-only attention as in the Medium model)."""
    from ..io.safetensors_io import save_file
    from ..models.dit_sd3 import random_sd3_weights
    from ..models.vae import random_vae_weights

    root = Path(root)
    dit = Sd3Config(pos_embed_max_size=48, num_attention_heads=4, attention_head_dim=64, num_layers=2,
                    joint_attention_dim=64, pooled_projection_dim=32, dual_attention_layers=(0,) if dual else ())
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_sd3_weights(dit, seed).items()},
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    from ..models.vae import random_vae_encoder_weights
    from .z_image import native_vae_encoder_to_diffusers

    vae_sd = native_vae_to_diffusers(random_vae_weights(vae, seed + 1), len(vae.ch_mult))
    vae_sd.update(native_vae_encoder_to_diffusers(random_vae_encoder_weights(vae, seed + 3)))
    save_file({k: v.bfloat16() for k, v in vae_sd.items()}, root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": {"pos_embed_max_size": dit.pos_embed_max_size, "num_attention_heads": dit.num_attention_heads,
                "attention_head_dim": dit.attention_head_dim, "num_layers": dit.num_layers,
                "joint_attention_dim": dit.joint_attention_dim, "pooled_projection_dim": dit.pooled_projection_dim,
                "dual_attention_layers": list(dit.dual_attention_layers)},
        "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks}, "text": "hash"}))
    return root
