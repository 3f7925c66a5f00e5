"""SANA providers `sana_1600m` and `sana_sprint_1600m` (and `cpu_*` on the fp32 oracle backend)
(parity: candle-gen-sana/src/model.rs, pipeline.rs, text_encoder.rs).

`sana_1600m`: Gemma-2-2b caption features (the prompt behind a fixed "complex human instruction", first token plus the
last 299 positions of the padded sequence -> [1, 300, 2304]), 20 flow-match Euler steps over the static-shift-3 table,
the trunk sees sigma * 1000, true classifier-free guidance 4.5 with the empty prompt as the negative; 32-channel
latents at 1/32 resolution decoded by the DC-AE after division by 0.41407.
`sana_sprint_1600m`: the same trunk distilled for 1-4 steps with the continuous-time-consistency (TrigFlow) sampler;
guidance (4.5) enters as an embedding (scale 0.1), there is no negative prompt.

Snapshot layout (diffusers): `transformer/`, `text_encoder/` + `tokenizer/tokenizer.json`, `vae/`."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..contracts.gen_core.generator import GenerationRequest
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import ScmScheduler, TorchLatentOps, build_flow_sigmas, run_scm_sampler
from ..models.dit_sana import DcAeConfig, DcAeDecoder, SanaConfig, SanaDiT, random_dcae_weights, random_sana_weights
from .family import FamilyPipeline, HashPromptEncoder, Variant, family_registrations, rgb8_image
from .seed import default_seed, for_each_image_seed

SHIFT = 3.0
MAX_SEQUENCE_LENGTH = 300
SANA_CHI_PROMPT = (
    "Given a user prompt, generate an 'Enhanced prompt' that provides detailed visual descriptions suitable for image "
    "generation. Evaluate the level of detail in the user prompt:\n- If the prompt is simple, focus on adding specifics "
    "about colors, shapes, sizes, textures, and spatial relationships to create vivid and concrete scenes.\n- If the "
    "prompt is already detailed, refine and enhance the existing details slightly without overcomplicating.\nHere are "
    "examples of how to transform or refine prompts:\n- User Prompt: A cat sleeping -> Enhanced: A small, fluffy white "
    "cat curled up in a round shape, sleeping peacefully on a warm sunny windowsill, surrounded by pots of blooming red "
    "flowers.\n- User Prompt: A busy city street -> Enhanced: A bustling city street scene at dusk, featuring glowing "
    "street lamps, a diverse crowd of people in colorful clothing, and a double-decker bus passing by towering glass "
    "skyscrapers.\nPlease generate only the enhanced description for the prompt below and avoid including any additional "
    "commentary or evaluations:\nUser Prompt: ")

VARIANTS = [
    Variant("sana_1600m", "sana", 20, 4.5, size_multiple=32, extra={"config": "base", "quants": True}),
    Variant("sana_sprint_1600m", "sana", 2, 4.5, size_multiple=32, embedded_guidance=True, fixed_sampler=True,
            extra={"config": "sprint"}),
]


class GemmaCaptionEncoder:
    """CHI prefix + prompt, right-padded to (prefix tokens + 300 - 2), through Gemma-2 with padding masked; the caption
    is position 0 followed by the last 299 positions of the padded sequence."""

    def __init__(self, lm, tokenizer, pad_id: int, max_len: int = MAX_SEQUENCE_LENGTH):
        self.lm, self.tok, self.pad_id, self.max_len = lm, tokenizer, pad_id, max_len
        self.prefix_tokens = len(tokenizer.encode(SANA_CHI_PROMPT).ids)

    def encode(self, prompt: str) -> torch.Tensor:
        total = self.prefix_tokens + self.max_len - 2
        ids = self.tok.encode(SANA_CHI_PROMPT + prompt.lower().strip()).ids[:total]
        n = len(ids)
        full = ids + [self.pad_id] * (total - n)
        S = len(full)
        j = torch.arange(S)
        allowed = ((j[None, :] <= j[:, None]) & (j[None, :] < n)) | (torch.eye(S, dtype=torch.bool) & (j[None, :] >= n))
        mask = torch.zeros(S, S).masked_fill(~allowed, float("-inf"))[None, None]
        h = self.lm.hidden_states(torch.tensor([full]), None, additive_mask=mask.to(self.lm.device, self.lm.dtype))
        h = self.lm._norm(h, "model.norm.weight")
        sel = [0] + list(range(S - self.max_len + 1, S))
        return h[:, sel]


@dataclass
class _Heavy:
    dit: SanaDiT
    vae: DcAeDecoder


class SanaPipeline(FamilyPipeline):
    latent_channels = 32
    latent_downscale = 32

    def __init__(self, variant, root, backend, device):
        super().__init__(variant, root, backend, device)
        self.dit_cfg = SanaConfig.sprint() if variant.extra["config"] == "sprint" else SanaConfig()
        self.vae_cfg = DcAeConfig()
        if "dit" in self.raw:
            self.dit_cfg = SanaConfig.from_json({**self.raw["dit"], "guidance_embeds": self.dit_cfg.guidance_embeds,
                                                 "qk_norm": self.dit_cfg.qk_norm})
        if "vae" in self.raw:
            self.vae_cfg = DcAeConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in self.raw["vae"].items()})
        self.latent_channels = self.dit_cfg.in_channels
        self.latent_downscale = self.vae_cfg.compression

    def load_text(self):
        if self.text_kind == "hash":
            h = HashPromptEncoder(self.dit_cfg.caption_channels, self.device, self.dtype)
            n = int(self.raw.get("caption_tokens", MAX_SEQUENCE_LENGTH))

            class _Fixed:
                def encode(self, prompt: str):
                    return h.encode(prompt, n).txt
            return _Fixed()
        import tokenizers

        from ..io.safetensors_io import load_dir
        from ..models.config import ModelConfig
        from ..models.oracle import OracleLlama

        te, tk = self.root / "text_encoder", self.root / "tokenizer" / "tokenizer.json"
        if not te.is_dir() or not tk.exists():
            raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks text_encoder/ or tokenizer/tokenizer.json")
        top = json.loads((te / "config.json").read_text())
        lm = OracleLlama(ModelConfig.from_json(top), load_dir(te), self.dtype, self.device)
        return GemmaCaptionEncoder(lm, tokenizers.Tokenizer.from_file(str(tk)), int(top.get("pad_token_id") or 0))

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir

        if self.random_init is not None:
            seed = int(self.random_init)
            dit_w, vae_w = random_sana_weights(self.dit_cfg, seed, 0.02), random_dcae_weights(self.vae_cfg, seed + 1)
        else:
            for d in ("transformer", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {d}/")
            dit_w, vae_w = load_dir(self.root / "transformer"), load_dir(self.root / "vae")
        # the decoder stays fp32 (deep stack of unnormalised residual convolutions; the reference runs it in f32 too)
        return _Heavy(SanaDiT(self.dit_cfg, dit_w, self.dtype, self.device),
                      DcAeDecoder(self.vae_cfg, vae_w, torch.float32, self.device))

    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        return build_flow_sigmas(steps, math.log(SHIFT))

    def scheduler_mu(self, req):
        return req.scheduler_shift if req.scheduler_shift is not None else math.log(SHIFT)

    def encode(self, text, req: GenerationRequest):
        def one(prompt):
            return {"cap": text.encode(prompt), "proj": None}

        g = self.guidance(req)
        return one(req.prompt), (one(req.negative_prompt or "") if self.cfg_active(g) else None)

    def _projected(self, heavy, cond):
        if cond["proj"] is None:
            cond["proj"] = heavy.dit.caption(cond["cap"])
        return cond["proj"]

    def velocity(self, heavy: _Heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        t = torch.full((x.shape[0],), sigma * 1000.0, device=self.device)
        return heavy.dit.forward(x, self._projected(heavy, cond), t, projected=True)

    def decode(self, heavy: _Heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        img = heavy.vae.decode(z.float() / self.vae_cfg.scaling_factor)[0]
        return [rgb8_image(img, req.width, req.height)]

    def render(self, heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        if not self.variant.embedded_guidance:
            return super().render(heavy, cond, req, on_progress)
        # SANA-Sprint: consistency sampling, one forward per step, guidance as an embedding
        steps = req.steps or self.variant.default_steps
        g = self.guidance(req)
        base_seed = req.seed if req.seed is not None else default_seed()
        sched = ScmScheduler.new(steps)
        ops = TorchLatentOps()
        gvec = torch.full((1,), float(g) * self.dit_cfg.guidance_embeds_scale, device=self.device)
        cap = self._projected(heavy, cond[0])

        def one_image(seed: int):
            x = self.initial_latent(seed, req).to(self.device, torch.float32)

            def on_step(i, n):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{self.variant.id}: cancelled at step {i}")
                on_progress(ProgressStep(i, n))

            def predict(x_in, scm_t):
                t = torch.full((1,), scm_t, device=self.device)
                return heavy.dit.forward(x_in.to(self.dtype), cap, t, gvec, projected=True).float()

            z = run_scm_sampler(ops, sched, x, seed, predict, on_step)
            if req.cancel.is_cancelled():
                raise Canceled(f"{self.variant.id}: cancelled before decode")
            on_progress(ProgressDecoding())
            return self.decode(heavy, z, req)

        return [img for imgs in for_each_image_seed(base_seed, req.count, one_image) for img in imgs]

    def validate(self, req: GenerationRequest) -> None:
        if self.variant.embedded_guidance and (req.sampler or req.scheduler):
            raise InferenceError(f"{self.variant.id}: the consistency sampler takes no sampler / scheduler choice")


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, SanaPipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0, sprint: bool = False) -> Path:
    """A tiny random SANA-shaped snapshot (hash caption encoder). The checkpoint carries the Sprint superset of keys
    (guidance embedder, q / k norms) under both timestep-embedder spellings, so either variant loads it."""
    from ..io.safetensors_io import save_file

    root = Path(root)
    base = dict(num_attention_heads=2, attention_head_dim=8, num_layers=2, num_cross_attention_heads=2,
                cross_attention_head_dim=8, caption_channels=24, in_channels=8, out_channels=8)
    vae = DcAeConfig(latent_channels=8, attention_head_dim=8, block_out_channels=(16, 16, 32, 32),
                     layers_per_block=(1, 1, 1, 1), block_types=("res", "res", "res", "evit"), qkv_multiscales=(3,))
    w = random_sana_weights(SanaConfig(**base, guidance_embeds=True, qk_norm=True), seed)
    for k in list(w):
        if k.startswith("time_embed.timestep_embedder."):
            w["time_embed.emb." + k[len("time_embed."):]] = w[k]
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.float() for k, v in w.items()}, root / "transformer" / "diffusion_pytorch_model.safetensors")
    save_file(random_dcae_weights(vae, seed + 1), root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": base, "text": "hash", "caption_tokens": 12,
        "vae": {"latent_channels": 8, "attention_head_dim": 8, "block_out_channels": [16, 16, 32, 32],
                "layers_per_block": [1, 1, 1, 1], "block_types": ["res", "res", "res", "evit"], "qkv_multiscales": [3]}}))
    return root
