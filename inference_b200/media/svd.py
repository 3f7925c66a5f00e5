"""Stable Video Diffusion image-to-video provider `svd_xt` (and `cpu_svd_xt`)
(parity: candle-gen-svd/src/lib.rs, pipeline.rs, preprocess.rs, scheduler.rs, image_encoder.rs).

One Reference image drives everything: its CLIP ViT-H embedding (antialiased resize to 224) is the UNet's single
cross-attention token, and its autoencoder latent (Lanczos resize to the output size, plus seeded noise of strength
`noise_aug_strength`, posterior mode, unscaled) is repeated per frame and concatenated to the noisy latents. The
request supplies frames (25), steps (25), conditioning fps (7; the UNet sees fps - 1), motion bucket (127), noise
augmentation (0.02), decode chunk size and the guidance ceiling (3.0): guidance ramps linearly over the frames from 1
to the ceiling and the unconditional branch zeroes both the embedding and the image latent. Sampling is EDM
v-prediction over a Karras table (sigma 700 -> 0.002, rho 7) with timestep 0.25 ln(sigma). There is no prompt.

Snapshot layout (diffusers): `unet/`, `vae/`, `image_encoder/`."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..contracts.gen_core import imageops
from ..contracts.gen_core.generator import ConditioningKind, GenerationRequest, Modality
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import EdmModelSampling, TorchLatentOps, denoise, get_solver
from ..models.unet_svd import (SvdUnet, SvdUnetConfig, SvdVae, SvdVaeConfig, karras_sigmas, random_svd_unet_weights,
                               random_svd_vae_weights)
from ..models.vision import CLIP_MEAN, CLIP_STD, VisionConfig, VisionTower
from .family import FamilyPipeline, Variant, family_registrations, video_frames_rgb8
from .seed import default_seed, seeded_normal

DEFAULT_FRAMES, DEFAULT_STEPS, DEFAULT_CONDITIONING_FPS, DEFAULT_FPS = 25, 25, 7, 7
MAX_FRAMES, MAX_STEPS, MAX_REFERENCE_DIM, SIZE_ALIGN = 64, 200, 8192, 64
VARIANTS = [Variant("svd_xt", "svd", DEFAULT_STEPS, 3.0, modality=Modality.VIDEO, conditioning=(ConditioningKind.REFERENCE,),
                    size_multiple=SIZE_ALIGN, min_size=SIZE_ALIGN, max_size=2048, max_count=1,
                    extra={"promptless": True, "no_negative": True})]


def clip_pixels(img: Image, size: int) -> torch.Tensor:
    """Antialiased bicubic resize of the whole image to size x size in [0, 1], then CLIP normalisation."""
    x = torch.frombuffer(bytearray(img.pixels), dtype=torch.uint8).view(img.height, img.width, 3).permute(2, 0, 1)[None].float() / 255.0
    x = torch.nn.functional.interpolate(x, size=(size, size), mode="bicubic", align_corners=False, antialias=True).clamp(0, 1)
    return (x - torch.tensor(CLIP_MEAN).view(1, 3, 1, 1)) / torch.tensor(CLIP_STD).view(1, 3, 1, 1)


@dataclass
class _Heavy:
    unet: SvdUnet
    vae: SvdVae


class SvdPipeline(FamilyPipeline):
    latent_channels = 4

    def __init__(self, variant, root, backend, device):
        super().__init__(variant, root, backend, device)
        self.dtype = torch.float32                       # every component runs fp32 (see models/unet_svd.py)
        rd = lambda d: json.loads((self.root / d / "config.json").read_text()) if (self.root / d / "config.json").exists() else {}   # noqa: E731
        self.unet_cfg = SvdUnetConfig.from_json(self.raw.get("unet", rd("unet")))
        self.vae_cfg = SvdVaeConfig.from_json(self.raw.get("vae", rd("vae")))
        enc = self.raw.get("image_encoder", rd("image_encoder"))
        self.enc_cfg = VisionConfig.from_json({"hidden_size": 1280, "intermediate_size": 5120, "num_hidden_layers": 32,
                                               "num_attention_heads": 16, "projection_dim": 1024, "hidden_act": "gelu", **enc}, "clip")

    def load_text(self):
        """The conditioning encoders: CLIP vision tower and the autoencoder (its encoder half is used here)."""
        from ..io.safetensors_io import load_dir

        if self.random_init is not None:
            raise LoadError(f"{self.variant.id}: random_init is not supported (the image encoder needs weights)")
        for d in ("image_encoder", "vae"):
            if not (self.root / d).is_dir():
                raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {d}/")
        tower = VisionTower(self.enc_cfg, load_dir(self.root / "image_encoder"), self.device, torch.float32)
        vae = SvdVae(self.vae_cfg, load_dir(self.root / "vae"), torch.float32, self.device)
        return tower, vae

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir

        if not (self.root / "unet").is_dir():
            raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks unet/")
        return _Heavy(SvdUnet(self.unet_cfg, load_dir(self.root / "unet"), torch.float32, self.device),
                      SvdVae(self.vae_cfg, load_dir(self.root / "vae"), torch.float32, self.device))

    # ---- request -------------------------------------------------------------------------------------------------
    def reference(self, req: GenerationRequest) -> Image:
        for c in req.conditioning:
            if c.kind is ConditioningKind.REFERENCE and c.image is not None:
                return c.image
        raise InferenceError(f"{self.variant.id}: image -> video requires a Reference image")

    def frames(self, req):
        return req.frames or DEFAULT_FRAMES

    def output_fps(self, req):
        return req.fps or DEFAULT_FPS

    def validate(self, req: GenerationRequest) -> None:
        mid = self.variant.id
        img = self.reference(req)
        if img.width == 0 or img.height == 0 or max(img.width, img.height) > MAX_REFERENCE_DIM:
            raise InferenceError(f"{mid}: reference image {img.width}x{img.height} outside 1..={MAX_REFERENCE_DIM}")
        if not 1 <= self.frames(req) <= MAX_FRAMES:
            raise InferenceError(f"{mid}: frames must be in 1..={MAX_FRAMES}")
        if req.steps is not None and not 1 <= req.steps <= MAX_STEPS:
            raise InferenceError(f"{mid}: steps must be in 1..={MAX_STEPS}")
        if req.decode_chunk_size is not None and req.decode_chunk_size < 1:
            raise InferenceError(f"{mid}: decode_chunk_size must be >= 1")
        if req.noise_aug_strength is not None and req.noise_aug_strength < 0:
            raise InferenceError(f"{mid}: noise_aug_strength must be >= 0")
        if req.conditioning_fps is not None and req.conditioning_fps < 1:
            raise InferenceError(f"{mid}: conditioning_fps must be >= 1")

    def encode(self, text, req: GenerationRequest):
        tower, vae = text
        img, F_ = self.reference(req), self.frames(req)
        seed = req.seed if req.seed is not None else default_seed()
        embeds = tower.image_embeds(clip_pixels(img, self.enc_cfg.image_size).to(self.device)).float()[:, None, :]
        rs = imageops.resize(img, req.width, req.height, "lanczos")
        x = torch.frombuffer(bytearray(rs.pixels), dtype=torch.uint8).view(req.height, req.width, 3).permute(2, 0, 1)[None].float() / 255.0
        aug = req.noise_aug_strength if req.noise_aug_strength is not None else 0.02
        noise = seeded_normal((seed + 7) % (1 << 64), 3 * req.height * req.width).view(1, 3, req.height, req.width)
        lat = vae.encode_mode((x * 2 - 1 + noise * aug).to(self.device))
        ids = torch.tensor([[float((req.conditioning_fps or DEFAULT_CONDITIONING_FPS) - 1),
                             req.motion_bucket_id if req.motion_bucket_id is not None else 127.0, aug]])
        return {"embeds": embeds, "latent": lat[:, None].expand(-1, F_, -1, -1, -1).contiguous(), "ids": ids, "seed": seed}, None

    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        c, _ = cond
        v, dev = self.variant, self.device
        steps, F_ = req.steps or v.default_steps, self.frames(req)
        max_g = req.guidance if req.guidance is not None else v.default_guidance
        sigmas = karras_sigmas(steps)
        ms, ops, solver = EdmModelSampling(0.002, 700.0), TorchLatentOps(), get_solver(req.sampler or "euler")
        h, w = req.height // 8, req.width // 8
        x = seeded_normal(c["seed"], F_ * 4 * h * w).view(1, F_, 4, h, w).to(dev) * (sigmas[0] ** 2 + 1.0) ** 0.5
        guide = torch.linspace(1.0, max_g, F_, device=dev).view(1, F_, 1, 1, 1) if F_ > 1 else torch.full((1, 1, 1, 1, 1), 1.0, device=dev)
        state = {"step": 0}

        def run_model(x_in, t):
            if req.cancel.is_cancelled():
                raise Canceled(f"{v.id}: cancelled at step {state['step']}")
            pos = heavy.unet.forward(torch.cat([x_in, c["latent"]], 2), t, c["embeds"], c["ids"])
            if max_g > 1.0:
                neg = heavy.unet.forward(torch.cat([x_in, torch.zeros_like(c["latent"])], 2), t, torch.zeros_like(c["embeds"]), c["ids"])
                pos = neg + guide * (pos - neg)
            state["step"] += 1
            if state["step"] <= steps:
                on_progress(ProgressStep(state["step"], steps))
            return pos

        x = solver.sample(ops, ms, lambda xx, s: denoise(ops, ms, xx, s, run_model), x, sigmas, c["seed"])
        while state["step"] < steps:
            state["step"] += 1
            on_progress(ProgressStep(state["step"], steps))
        if req.cancel.is_cancelled():
            raise Canceled(f"{v.id}: cancelled before decode")
        on_progress(ProgressDecoding())
        z = x[0] / self.vae_cfg.scaling_factor
        chunk = max(1, req.decode_chunk_size or F_)
        video = torch.cat([heavy.vae.decode(z[s:s + chunk], min(chunk, F_ - s)) for s in range(0, F_, chunk)], 0)   # [F, 3, H, W]
        return video_frames_rgb8(video.permute(1, 0, 2, 3), req.width, req.height)


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, SvdPipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random SVD-shaped snapshot in the diffusers layout (with a small CLIP vision tower)."""
    from ..io.safetensors_io import save_file
    from ..models.vision import random_vision_weights

    root = Path(root)
    unet = SvdUnetConfig(block_out_channels=(8, 16), num_attention_heads=(2, 2), cross_attention_dim=12,
                         addition_time_embed_dim=4, projection_class_embeddings_input_dim=12, groups=4)
    vae = SvdVaeConfig(block_out_channels=(8, 8, 8, 16), layers_per_block=1, groups=4)
    enc = dict(hidden_size=16, intermediate_size=32, num_hidden_layers=2, num_attention_heads=2, image_size=28, patch_size=14,
               projection_dim=12, hidden_act="gelu")
    for d in ("unet", "vae", "image_encoder"):
        (root / d).mkdir(parents=True, exist_ok=True)
    save_file(random_svd_unet_weights(unet, seed), root / "unet" / "diffusion_pytorch_model.safetensors")
    save_file(random_svd_vae_weights(vae, seed + 1), root / "vae" / "diffusion_pytorch_model.safetensors")
    save_file(random_vision_weights(VisionConfig.from_json(enc, "clip"), seed + 2), root / "image_encoder" / "model.safetensors")
    tj = lambda c, cls: {k: (list(x) if isinstance(x := getattr(c, k), tuple) else x) for k in cls.__dataclass_fields__}   # noqa: E731
    (root / "swb_config.json").write_text(json.dumps({"unet": tj(unet, SvdUnetConfig), "vae": tj(vae, SvdVaeConfig), "image_encoder": enc}))
    return root
