"""Stable Diffusion XL provider `sdxl` (and `cpu_sdxl` on the fp32 backend)
(parity: candle-gen-sdxl/src/lib.rs, pipeline.rs, conditioning.rs, denoise.rs).

Conditioning: CLIP-L and OpenCLIP-bigG second-to-last hidden states side by side -> context [77, 2048]; the bigG
projected pooled vector [1280] plus six size / crop numbers feed the UNet's additional embedding. Sampling is
noise-prediction over the scaled-linear DDPM table through the shared solver / schedule framework (default `ddim`
over the `normal` schedule, 30 steps), classifier-free guidance 7.0 with the encoded negative prompt (empty by
default). Latents are 4-channel at 1/8 resolution; the VAE is the SDXL autoencoder (scaling 0.13025, no shift).

Snapshot layout (diffusers): `unet/`, `text_encoder/` + `tokenizer/`, `text_encoder_2/` + `tokenizer_2/`, `vae/`;
`swb_config.json` overrides dimensions for synthetic snapshots."""
from __future__ import annotations

import dataclasses
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
from ..contracts.gen_core.sampling import (SCHEDULERS, SOLVERS, DiscreteModelSampling, TorchLatentOps, denoise, get_solver,
                                           schedule_sigmas)
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.unet_sdxl import SdxlUnet, SdxlUnetConfig
from ..models.vae import OracleVaeDecoder, VaeConfig
from .chroma import convert_diffusers_vae_decoder, native_vae_to_diffusers
from .residency import Residency
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw

MODEL_ID = "sdxl"
DEFAULT_STEPS, DEFAULT_GUIDANCE, DEFAULT_SAMPLER, DEFAULT_SCHEDULER = 30, 7.0, "ddim", "normal"
VAE_SCALE = 0.13025
SIZE_MULTIPLE = 8


@dataclass
class SdxlConditioning:
    context: torch.Tensor        # [1, 77, 2048]
    pooled: torch.Tensor         # [1, 1280]


class DualClipEncoders:
    def __init__(self, clip_l, tok_l, clip_g, tok_g):
        self.clip_l, self.tok_l, self.clip_g, self.tok_g = clip_l, tok_l, clip_g, tok_g

    @staticmethod
    def from_snapshot(root: Path, backend: str, device) -> "DualClipEncoders":
        from ..models.text_encoders import ClipTextConfig, ClipTextEncoder
        from .text_models import ClipBpeTokenizer, _load_component

        dtype = torch.bfloat16 if backend == "b200" else torch.float32
        missing = [d for d in ("text_encoder", "text_encoder_2", "tokenizer", "tokenizer_2") if not (root / d).is_dir()]
        if missing:
            raise LoadError(f"sdxl snapshot {root}: missing text-encoder components {missing}")
        parts = []
        for enc, tok in (("text_encoder", "tokenizer"), ("text_encoder_2", "tokenizer_2")):
            cj, cw = _load_component(root / enc)
            cfg = ClipTextConfig.from_json(cj)
            parts += [ClipTextEncoder(cfg, cw, device, dtype), ClipBpeTokenizer.from_dir(root / tok, cfg.max_position_embeddings)]
        return DualClipEncoders(*parts)

    def encode(self, prompt: str) -> SdxlConditioning:
        l = self.clip_l.encode_all(torch.tensor([self.tok_l.encode(prompt)], dtype=torch.int64))
        g = self.clip_g.encode_all(torch.tensor([self.tok_g.encode(prompt, pad_id=0)], dtype=torch.int64))
        return SdxlConditioning(torch.cat([l["penultimate"], g["penultimate"]], -1), g.get("projected", g["pooled"]))


class HashDualEncoders:
    def __init__(self, width: int, pooled: int, device, dtype):
        from .text_encoders import HashTextEncoders

        self.h = HashTextEncoders(width, pooled, device, dtype)

    def encode(self, prompt: str) -> SdxlConditioning:
        c = self.h.encode(prompt, 16)
        return SdxlConditioning(c.txt, c.pooled)


@dataclass
class _Heavy:
    unet: Any
    vae: Any
    post_quant: tuple[torch.Tensor, torch.Tensor] | None = None      # the autoencoder's 1x1 convolution in front of the decoder


def apply_post_quant(z: torch.Tensor, post_quant, cfg: VaeConfig) -> torch.Tensor:
    """The decoders compute conv_in(z / scale + shift); a checkpoint with `post_quant_conv` wants
    conv_in(pq(z / scale + shift)). Returns z' with z' / scale + shift == pq(z / scale + shift)."""
    if post_quant is None:
        return z
    w, b = post_quant
    u = torch.nn.functional.conv2d(z.float() / cfg.scale_factor + cfg.shift_factor, w.float().to(z.device), b.float().to(z.device))
    return (u - cfg.shift_factor) * cfg.scale_factor


class SdxlPipeline:
    model_id, default_steps, default_guidance = MODEL_ID, DEFAULT_STEPS, DEFAULT_GUIDANCE
    default_sampler, default_scheduler = DEFAULT_SAMPLER, DEFAULT_SCHEDULER

    @staticmethod
    def default_unet_config() -> SdxlUnetConfig:
        return SdxlUnetConfig()

    @staticmethod
    def model_sampling() -> DiscreteModelSampling:
        return DiscreteModelSampling()

    def __init__(self, root: Path, backend: str, device: torch.device):
        self.root, self.backend, self.device = Path(root), backend, device
        self.unet_cfg = self.default_unet_config()
        self.vae_cfg = VaeConfig(z_channels=4, scale_factor=VAE_SCALE, shift_factor=0.0)
        self.text_kind, self.random_init, self.adapters = "dual_clip", None, []
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            raw = json.loads(cfg_path.read_text())
            if "unet" in raw:
                u = dict(raw["unet"])
                for k in ("block_out_channels", "transformer_layers_per_block"):
                    if k in u:
                        u[k] = tuple(u[k])
                self.unet_cfg = dataclasses.replace(self.default_unet_config(), **u)
            if "vae" in raw:
                v = dict(raw["vae"])
                if "ch_mult" in v:
                    v["ch_mult"] = tuple(v["ch_mult"])
                self.vae_cfg = VaeConfig(**{"z_channels": 4, "scale_factor": VAE_SCALE, "shift_factor": 0.0, **v})
            self.text_kind = raw.get("text", self.text_kind)
            self.random_init = raw.get("random_init")
        elif (self.root / "unet" / "config.json").exists():
            self.unet_cfg = SdxlUnetConfig.from_json(json.loads((self.root / "unet" / "config.json").read_text()))
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32

    def load_text(self):
        if self.text_kind == "hash":
            pooled = self.unet_cfg.projection_class_embeddings_input_dim - 6 * self.unet_cfg.addition_time_embed_dim
            return HashDualEncoders(self.unet_cfg.cross_attention_dim, pooled, self.device, self.dtype)
        return DualClipEncoders.from_snapshot(self.root, self.backend, self.device)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir, load_file
        from ..models.unet_sdxl import random_sdxl_unet_weights
        from ..models.vae import random_vae_weights

        gpu = self.backend == "b200"
        pq = None
        if self.random_init is not None and gpu:
            seed = int(self.random_init)
            unet_w = random_sdxl_unet_weights(self.unet_cfg, seed, 0.02, torch.bfloat16, self.device)
            vae_w = random_vae_weights(self.vae_cfg, seed + 1, dtype=torch.bfloat16, device=self.device)
        else:
            for d in ("unet", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks {d}/")
            unet_w = load_dir(self.root / "unet")
            for ad in self.adapters:
                from .train import merge_lora

                if not Path(ad.path).is_file():
                    raise LoadError(f"{MODEL_ID}: adapter file {ad.path} not found")
                unet_w = merge_lora(unet_w, load_file(ad.path), ad.scale if ad.scale is not None else 1.0, prefix="unet.")
            raw_vae = load_dir(self.root / "vae")
            vae_w = convert_diffusers_vae_decoder(raw_vae, len(self.vae_cfg.ch_mult))
            if "post_quant_conv.weight" in raw_vae:
                pq = (raw_vae["post_quant_conv.weight"], raw_vae["post_quant_conv.bias"])
        unet = SdxlUnet(self.unet_cfg, unet_w, self.dtype, self.device)
        if gpu:
            from ..models.vae import VaeDecoderGpu

            # the device decoder's convolutions are GEMMs whose reduction size must be a multiple of 8: the 4 latent
            # channels are padded to 8 with zero weights (render pads the latents with zero channels; the shift is 0)
            pad = (-self.vae_cfg.z_channels) % 8
            vae_w = dict(vae_w)
            vae_w["decoder.conv_in.weight"] = torch.nn.functional.pad(vae_w["decoder.conv_in.weight"], (0, 0, 0, 0, 0, pad))
            gpu_cfg = dataclasses.replace(self.vae_cfg, z_channels=self.vae_cfg.z_channels + pad)
            return _Heavy(unet, VaeDecoderGpu(gpu_cfg, self.device).load_state_dict(vae_w), pq)
        return _Heavy(unet, OracleVaeDecoder(self.vae_cfg, vae_w, device=self.device), pq)

    def guidance(self, req: GenerationRequest) -> float:
        return float(req.guidance) if req.guidance is not None else self.default_guidance

    def encode(self, text, req: GenerationRequest):
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt or "") if self.guidance(req) > 1.0 else None
        return pos, neg

    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        steps = req.steps or self.default_steps
        guidance = self.guidance(req)
        base_seed = req.seed if req.seed is not None else default_seed()
        lh, lw = req.height // 8, req.width // 8
        dev, dt = self.device, self.dtype
        ms = self.model_sampling()
        sigmas = schedule_sigmas(req.scheduler or self.default_scheduler, ms, steps)
        solver, ops = get_solver(req.sampler or self.default_sampler), TorchLatentOps()
        from .chroma import convert_diffusers_vae_encoder
        from .reference import encode_reference_image, init_time_step, reference_of

        ref = reference_of(req, self.model_id)
        clean, start = None, 0
        if ref is not None and init_time_step(steps, ref[1]) > 0:
            from ..io.safetensors_io import load_dir

            raw = load_dir(self.root / "vae")
            enc_w = convert_diffusers_vae_encoder(raw)
            enc_w.update({k: t for k, t in raw.items() if k.startswith("quant_conv.")})
            start = min(init_time_step(steps, ref[1]), len(sigmas) - 2)
            clean = encode_reference_image(self.vae_cfg, enc_w, ref[0], req.width, req.height, dev, self.model_id).to(dev)
            sigmas = sigmas[start:]                    # the run enters the schedule at sigma_start
        conds = [c for c in cond if c is not None]                 # [prompt] or [prompt, negative]
        context = torch.cat([c.context for c in conds], 0).to(dev, dt)
        pooled = torch.cat([c.pooled for c in conds], 0).to(dev, dt)
        nb = len(conds)
        time_ids = torch.tensor([[req.height, req.width, 0, 0, req.height, req.width]] * nb, dtype=torch.float32, device=dev)

        def one_image(seed: int) -> Image:
            k_noise, k_latent = ms.noise_scaling_coeffs(sigmas[0])
            x = seeded_noise_nchw(seed, self.vae_cfg.z_channels, lh, lw).to(dev) * k_noise
            if clean is not None:                       # variance-exploding form: clean + sigma * noise
                x = x.float() + k_latent * clean
            x = x.to(dt).contiguous()
            state = {"step": start}
            for s_done in range(1, start + 1):
                on_progress(ProgressStep(s_done, steps))

            def run_model(x_in, timestep):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{self.model_id}: cancelled at step {state['step']}")
                tt = torch.full((nb,), float(timestep), device=dev)
                o = heavy.unet.forward(x_in.expand(nb, -1, -1, -1), tt, context, pooled, time_ids).float()
                eps = o[0:1] if nb == 1 else o[1:2] + (o[0:1] - o[1:2]) * guidance
                state["step"] += 1
                if state["step"] <= steps:
                    on_progress(ProgressStep(state["step"], steps))
                return eps.to(dt).contiguous()

            x = solver.sample(ops, ms, lambda xx, s: denoise(ops, ms, xx, s, run_model), x, sigmas, seed)
            while state["step"] < steps:
                state["step"] += 1
                on_progress(ProgressStep(state["step"], steps))
            if req.cancel.is_cancelled():
                raise Canceled(f"{self.model_id}: cancelled before decode")
            on_progress(ProgressDecoding())
            z = apply_post_quant(x.float(), heavy.post_quant, self.vae_cfg)
            if self.backend == "b200":
                z = torch.nn.functional.pad(z, (0, 0, 0, 0, 0, heavy.vae.cfg.z_channels - z.shape[1]))
                host = heavy.vae.decode_rgb8(z)[0].cpu()
            else:
                img = heavy.vae.decode(z)[0].permute(1, 2, 0)
                host = torch.round((img.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).cpu()
            return Image(width=req.width, height=req.height, pixels=host.contiguous().numpy().tobytes())

        return for_each_image_seed(base_seed, req.count, one_image)


def sdxl_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family="sdxl", backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False,
            conditioning=[ConditioningKind.REFERENCE],
            supports_lora=True, supports_lokr=False, samplers=list(SOLVERS), schedulers=list(SCHEDULERS),
            supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8,
            supports_sequential_offload=True),
        required_components=[])


class SdxlGenerator(Generator):
    def __init__(self, pipe: SdxlPipeline, descriptor: ModelDescriptor, policy: OffloadPolicy):
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
        levels = len(self.pipe.unet_cfg.block_out_channels) - 1
        mult = SIZE_MULTIPLE << levels
        if req.width % mult or req.height % mult:
            raise InferenceError(f"{mid}: width/height must be multiples of {mult} (got {req.width}x{req.height})")

    def generate(self, req: GenerationRequest, on_progress: Callable = lambda p: None) -> GenerationOutput:
        self.validate(req)
        images = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(images=images)


def _load(backend: str, prefix: str) -> Callable[[LoadSpec], SdxlGenerator]:
    def load(spec: LoadSpec) -> SdxlGenerator:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise Unsupported(f"{mid}: needs a snapshot directory (single-file checkpoints: remap with "
                              "contracts.gen_core.sdxl_ldm and save in the directory layout)")
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
        pipe = SdxlPipeline(Path(spec.weights.path), backend, device)
        pipe.adapters = list(spec.adapters)
        return SdxlGenerator(pipe, sdxl_descriptor(backend, prefix), spec.offload_policy)
    return load


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=lambda: sdxl_descriptor(backend, prefix), load=_load(backend, prefix))]


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random SDXL-shaped snapshot in the diffusers directory layout with the weight-free prompt encoder."""
    from ..io.safetensors_io import save_file
    from ..models.unet_sdxl import random_sdxl_unet_weights
    from ..models.vae import random_vae_weights

    root = Path(root)
    unet = SdxlUnetConfig(block_out_channels=(32, 64, 128), transformer_layers_per_block=(0, 1, 2), attention_head_dim=64,
                          cross_attention_dim=64, addition_time_embed_dim=8, projection_class_embeddings_input_dim=32 + 48,
                          norm_groups=8)
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1, z_channels=4, scale_factor=VAE_SCALE, shift_factor=0.0)
    (root / "unet").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_sdxl_unet_weights(unet, seed).items()},
              root / "unet" / "diffusion_pytorch_model.safetensors")
    vae_sd = {k: v.bfloat16() for k, v in native_vae_to_diffusers(random_vae_weights(vae, seed + 1), len(vae.ch_mult)).items()}
    g = torch.Generator().manual_seed(seed + 2)
    vae_sd["post_quant_conv.weight"] = (torch.eye(4).view(4, 4, 1, 1) + 0.2 * torch.randn(4, 4, 1, 1, generator=g)).bfloat16()
    vae_sd["post_quant_conv.bias"] = (0.1 * torch.randn(4, generator=g)).bfloat16()
    from ..models.vae import random_vae_encoder_weights
    from .z_image import native_vae_encoder_to_diffusers

    vae_sd.update({k: t.bfloat16() for k, t in native_vae_encoder_to_diffusers(random_vae_encoder_weights(vae, seed + 3)).items()})
    vae_sd["quant_conv.weight"] = (torch.eye(8).view(8, 8, 1, 1) + 0.2 * torch.randn(8, 8, 1, 1, generator=g)).bfloat16()
    vae_sd["quant_conv.bias"] = (0.1 * torch.randn(8, generator=g)).bfloat16()
    save_file(vae_sd, root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "unet": {"block_out_channels": list(unet.block_out_channels),
                 "transformer_layers_per_block": list(unet.transformer_layers_per_block),
                 "attention_head_dim": unet.attention_head_dim, "cross_attention_dim": unet.cross_attention_dim,
                 "addition_time_embed_dim": unet.addition_time_embed_dim,
                 "projection_class_embeddings_input_dim": unet.projection_class_embeddings_input_dim,
                 "norm_groups": unet.norm_groups},
        "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks}, "text": "hash"}))
    return root
