"""Mochi 1 text-to-video provider `mochi_1` (and `cpu_mochi_1` on the fp32 oracle backend)
(parity: candle-gen-mochi/src/lib.rs, pipeline.rs, scheduler.rs, text_encoder.rs).

T5-XXL states of the prompt (at most 256 tokens, padding masked) condition a dual-stream DiT; true classifier-free
guidance (default 4.5, negative prompt default "") over 64 Euler steps of the linear-quadratic noise table; the
network's time input is (1 - noise level) * 1000 and it predicts the velocity towards the clean sample. Latents are
12-channel at 1/8 resolution and one latent frame per six video frames (clip lengths 6k + 1); the decoder runs in fp32,
frame-chunked, and the result is `frames` RGB8 images at 30 fps.

Snapshot layout: `transformer/`, `text_encoder/` + `tokenizer/` (`tokenizer.json` or `spiece.model`), `vae/`."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from ..contracts.errors import InferenceError, LoadError
from ..contracts.gen_core.generator import GenerationRequest, Modality
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..models.dit_mochi import (MochiConfig, MochiDiT, MochiVaeConfig, MochiVaeDecoder, linear_quadratic_sigmas,
                                random_mochi_vae_weights, random_mochi_weights)
from .family import FamilyPipeline, HashPromptEncoder, Variant, family_registrations, video_frames_rgb8
from .seed import seeded_noise_nchw

MAX_SEQUENCE_LENGTH, PAD_TOKEN_ID, EOS_TOKEN_ID = 256, 0, 1
DEFAULT_FRAMES, DEFAULT_FPS, DECODE_CHUNK_FRAMES = 19, 30, 1
VARIANTS = [Variant("mochi_1", "mochi", 64, 4.5, modality=Modality.VIDEO, size_multiple=16, min_size=16,
                    max_size=1280, max_count=1)]


class MochiPromptEncoder:
    """T5 over the prompt padded to 256 tokens with padding masked as keys; returns the valid rows."""

    def __init__(self, t5, encode_ids):
        self.t5, self.encode_ids = t5, encode_ids

    def encode(self, prompt: str) -> torch.Tensor:
        ids = list(self.encode_ids(prompt))
        if len(ids) > MAX_SEQUENCE_LENGTH:
            ids = ids[:MAX_SEQUENCE_LENGTH - 1] + [EOS_TOKEN_ID]
        n = len(ids)
        padded = torch.tensor([ids + [PAD_TOKEN_ID] * (MAX_SEQUENCE_LENGTH - n)], dtype=torch.int64)
        mask = torch.tensor([[1] * n + [0] * (MAX_SEQUENCE_LENGTH - n)])
        return self.t5.encode(padded, mask)[:, :n]


@dataclass
class _Heavy:
    dit: MochiDiT
    vae: MochiVaeDecoder


class MochiPipeline(FamilyPipeline):
    latent_channels = 12

    def __init__(self, variant, root, backend, device):
        super().__init__(variant, root, backend, device)
        self.dit_cfg = MochiConfig.from_json(self.raw["dit"]) if "dit" in self.raw else MochiConfig()
        self.vae_cfg = MochiVaeConfig()
        if "vae" in self.raw:
            self.vae_cfg = MochiVaeConfig.from_json(self.raw["vae"])
        elif (self.root / "vae" / "config.json").exists():
            self.vae_cfg = MochiVaeConfig.from_json(json.loads((self.root / "vae" / "config.json").read_text()))
        self.latent_channels = self.dit_cfg.in_channels

    def load_text(self):
        if self.text_kind == "hash":
            h = HashPromptEncoder(self.dit_cfg.text_embed_dim, self.device, self.dtype, min_len=1)

            class _Valid:
                def encode(self, prompt: str):
                    return h.encode(prompt, min(MAX_SEQUENCE_LENGTH, 1 + len(prompt.split()))).txt
            return _Valid()
        from ..models.text_encoders import T5Config, T5Encoder
        from .text_models import T5SentencePieceTokenizer, _load_component

        te, tk = self.root / "text_encoder", self.root / "tokenizer"
        if not te.is_dir() or not tk.is_dir():
            raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks text_encoder/ or tokenizer/")
        if (tk / "tokenizer.json").exists():
            import tokenizers

            tok = tokenizers.Tokenizer.from_file(str(tk / "tokenizer.json"))
            tok.no_padding()
            enc = lambda p: tok.encode(p, add_special_tokens=True).ids       # noqa: E731
        elif (tk / "spiece.model").exists():
            sp = T5SentencePieceTokenizer(tk / "spiece.model")
            enc = lambda p: sp.sp.encode(p) + [sp.eos]                        # noqa: E731
        else:
            raise LoadError(f"{self.variant.id}: {tk} has neither tokenizer.json nor spiece.model")
        cfg, w = _load_component(te)
        return MochiPromptEncoder(T5Encoder(T5Config.from_json(cfg), w, self.device, self.dtype), enc)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir

        if self.random_init is not None:
            seed = int(self.random_init)
            dit_w, vae_w = random_mochi_weights(self.dit_cfg, seed, 0.02), random_mochi_vae_weights(self.vae_cfg, seed + 1)
        else:
            for d in ("transformer", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {d}/")
            dit_w, vae_w = load_dir(self.root / "transformer"), load_dir(self.root / "vae")
        return _Heavy(MochiDiT(self.dit_cfg, dit_w, self.dtype, self.device),
                      MochiVaeDecoder(self.vae_cfg, vae_w, torch.float32, self.device))

    # ---- request shape -----------------------------------------------------------------------------------------------
    def frames(self, req: GenerationRequest) -> int:
        return req.frames or DEFAULT_FRAMES

    def output_fps(self, req: GenerationRequest) -> int:
        return req.fps or DEFAULT_FPS

    def validate(self, req: GenerationRequest) -> None:
        f, r = self.frames(req), self.vae_cfg.temporal_ratio
        if (f - 1) % r:
            raise InferenceError(f"{self.variant.id}: frames must be {r}k + 1 (got {f})")
        if req.steps is not None and req.steps < 2:
            raise InferenceError(f"{self.variant.id}: the linear-quadratic table needs at least 2 steps")

    def initial_latent(self, seed: int, req: GenerationRequest) -> torch.Tensor:
        lf = 1 + (self.frames(req) - 1) // self.vae_cfg.temporal_ratio
        s, C = self.vae_cfg.spatial_ratio, self.latent_channels
        return seeded_noise_nchw(seed, C * lf, req.height // s, req.width // s).reshape(1, C, lf, req.height // s, req.width // s)

    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        return linear_quadratic_sigmas(steps) + [0.0]

    def cfg_active(self, guidance) -> bool:
        return True                                   # the reference always evaluates the [negative, positive] pair

    def velocity(self, heavy: _Heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        t = torch.full((x.shape[0],), (1.0 - sigma) * 1000.0, device=self.device)
        return -heavy.dit.forward(x, cond, t)         # the network's velocity points at the clean sample

    def decode(self, heavy: _Heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        video = heavy.vae.decode(z.float(), DECODE_CHUNK_FRAMES)[0]
        return video_frames_rgb8(video[:, : self.frames(req)], req.width, req.height)


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, MochiPipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random Mochi-shaped snapshot (hash prompt features)."""
    from ..io.safetensors_io import save_file

    root = Path(root)
    dit = MochiConfig(num_heads=2, head_dim=16, num_layers=2, pooled_dim=24, text_embed_dim=16, time_embed_dim=16, pool_heads=2)
    vae = MochiVaeConfig(decoder_block_out_channels=(8, 8, 8, 16), layers_per_block=(1, 1, 1, 1, 1), groups=4)
    for d in ("transformer", "vae"):
        (root / d).mkdir(parents=True, exist_ok=True)
    save_file(random_mochi_weights(dit, seed), root / "transformer" / "diffusion_pytorch_model.safetensors")
    save_file(random_mochi_vae_weights(vae, seed + 1), root / "vae" / "diffusion_pytorch_model.safetensors")
    jd = {k: getattr(dit, k) for k in MochiConfig.__dataclass_fields__}
    jv = {k: (list(v) if isinstance(v := getattr(vae, k), tuple) else v) for k in MochiVaeConfig.__dataclass_fields__}
    (root / "swb_config.json").write_text(json.dumps({"dit": jd, "vae": jv, "text": "hash"}))
    return root
