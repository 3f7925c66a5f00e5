"""Ideogram 4 text-to-image providers `ideogram_4` and `ideogram_4_turbo` (and `cpu_*` on the fp32 oracle backend)
(parity: candle-gen-ideogram/src/lib.rs, pipeline.rs, scheduler.rs, adapters.rs).

The prompt goes through the language tower of Qwen3-VL-8B; the hidden states after 13 tapped depths (the embeddings,
every third layer up to 33, and 35) are interleaved on the feature axis (feature h of layer j sits at h * 13 + j).
Prompt rows and image rows form ONE sequence for a single-stream DiT. Model time runs from ~0 (noise) to ~1 (image)
along a resolution-aware logit-normal table; this module maps it onto the framework's sigma = 1 - t so the shared
solvers apply (dx / dsigma = -v).

`ideogram_4`: 48 steps, guidance 7: a second, unconditional DiT sees the image rows only, v = g v_cond + (1 - g)
v_uncond, and the last three steps use guidance 3. There is no negative prompt.
`ideogram_4_turbo`: the conditional DiT with the bundled TurboTime low-rank adapter (`turbo_lora.safetensors`) merged at
load; 8 steps, one forward per step, guidance inert.
Latents are FLUX.2's: 32 channels at 1/8 resolution packed 2 x 2 into 128-wide tokens (here in (row, column, channel)
order inside a patch), normalised by the autoencoder's batch-norm statistics.

Image-conditioned editing (a source image re-noised to a start time, optional inpaint mask) needs the autoencoder's
encoder and is not built here.

Snapshot layout: `transformer/`, `unconditional_transformer/`, `text_encoder/` + `tokenizer/tokenizer.json`, `vae/`,
`turbo_lora.safetensors`."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ..contracts.errors import InferenceError, LoadError
from ..contracts.gen_core.generator import GenerationRequest
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..models.dit_ideogram import (IdeogramConfig, IdeogramDiT, logit_normal_time, packing, preset_mu_std,
                                   random_ideogram_weights)
from ..models.vae import VaeConfig, random_vae_weights
from .family import HashPromptEncoder, Variant, family_registrations, load_vl_text_tower
from .flux2 import Flux2Pipeline

EXTRACTED_LAYERS = (0, 3, 6, 9, 12, 15, 18, 21, 24, 27, 30, 33, 35)
MAX_TEXT_TOKENS = 2048
POLISH_STEPS, POLISH_GUIDANCE = 3, 3.0
TURBO_LORA_FILE, TURBO_LORA_SCALE = "turbo_lora.safetensors", 1.0
LORA_PREFIXES = ("diffusion_model.", "transformer.", "model.")

VARIANTS = [
    Variant("ideogram_4", "ideogram", 48, 7.0, size_multiple=16, fixed_sampler=True, extra={"no_negative": True}),
    Variant("ideogram_4_turbo", "ideogram", 8, None, size_multiple=16, fixed_sampler=True, extra={"turbo": True}),
]
_UNCOND = "unconditional"


class IdeogramPromptEncoder:
    def __init__(self, encoder, tokenizer, select=EXTRACTED_LAYERS):
        self.encoder, self.tok, self.select = encoder, tokenizer, list(select)

    def encode(self, prompt: str) -> torch.Tensor:
        ids = self.tok.encode(prompt).ids[:MAX_TEXT_TOKENS]
        if not ids:
            raise InferenceError("ideogram: the prompt tokenised to nothing")
        h = self.encoder.encode_layers(ids, self.select)                      # [1, S, 13, H]
        return h.permute(0, 1, 3, 2).reshape(1, len(ids), -1)                 # layer index innermost


def normalise_lora(adapter: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Any of the accepted spellings (`lora_down` / `lora_up`, `lora_A` / `lora_B`, with or without `.weight`, under
    `diffusion_model.` / `transformer.` / `model.` or no prefix) -> `transformer.<module>.lora_{A,B}.weight`."""
    out = {}
    for k, v in adapter.items():
        for pre in LORA_PREFIXES:
            if k.startswith(pre):
                k = k[len(pre):]
                break
        k = k.replace(".lora_down", ".lora_A").replace(".lora_up", ".lora_B")
        if k.endswith((".lora_A", ".lora_B")):
            k += ".weight"
        out["transformer." + k] = v
    return out


@dataclass
class _Heavy:
    dit: IdeogramDiT
    uncond: IdeogramDiT | None
    vae: Any
    post_quant: tuple[torch.Tensor, torch.Tensor] | None
    bn_mean: torch.Tensor
    bn_std: torch.Tensor


class IdeogramPipeline(Flux2Pipeline):
    latent_channels = 128
    latent_downscale = 16

    def __init__(self, variant, root, backend, device):
        super(Flux2Pipeline, self).__init__(variant, root, backend, device)
        self.dit_cfg = IdeogramConfig.from_json(self.raw["dit"]) if "dit" in self.raw else IdeogramConfig()
        v = dict(self.raw.get("vae", {}))
        if "ch_mult" in v:
            v["ch_mult"] = tuple(v["ch_mult"])
        self.vae_cfg = VaeConfig(**{"z_channels": 32, "scale_factor": 1.0, "shift_factor": 0.0, **v})
        self.select = tuple(self.raw.get("te_layers", EXTRACTED_LAYERS))
        self.turbo = bool(variant.extra.get("turbo"))

    def load_text(self):
        if self.text_kind == "hash":
            return HashPromptEncoder(self.dit_cfg.llm_features_dim, self.device, self.dtype)
        enc, tok = load_vl_text_tower(self.variant.id, self.root, self.device, max(self.select))
        return IdeogramPromptEncoder(enc, tok, self.select)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir, load_file
        from .train import merge_lora

        uncond_w = None
        if self.random_init is not None:
            seed = int(self.random_init)
            dit_w = random_ideogram_weights(self.dit_cfg, seed, 0.02)
            if not self.turbo:
                uncond_w = random_ideogram_weights(self.dit_cfg, seed + 2, 0.02)
        else:
            need = ("transformer",) if self.turbo else ("transformer", "unconditional_transformer")
            for d in need:
                if not (self.root / d).is_dir():
                    raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {d}/")
            dit_w = load_dir(self.root / "transformer")
            if self.turbo:
                lora = self.root / TURBO_LORA_FILE
                if not lora.is_file():
                    raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {TURBO_LORA_FILE}")
                dit_w = merge_lora(dit_w, normalise_lora(load_file(lora)), TURBO_LORA_SCALE)
            else:
                uncond_w = load_dir(self.root / "unconditional_transformer")
        dit = IdeogramDiT(self.dit_cfg, dit_w, self.dtype, self.device)
        uncond = IdeogramDiT(self.dit_cfg, uncond_w, self.dtype, self.device) if uncond_w is not None else None
        return _Heavy(dit, uncond, *self.load_vae())

    # ---- schedule ----------------------------------------------------------------------------------------------------
    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        mu, std = preset_mu_std(steps)
        return [1.0 - logit_normal_time(1.0 - i / steps, req.height, req.width, mu, std) for i in range(steps + 1)]

    def cfg_active(self, guidance) -> bool:
        return not self.turbo

    def step_guidance(self, step: int, steps: int, guidance: float) -> float:
        return POLISH_GUIDANCE if step >= steps - POLISH_STEPS else guidance

    def encode(self, text, req: GenerationRequest):
        feats = text.encode(req.prompt)
        feats = feats.txt if hasattr(feats, "txt") else feats
        return feats, (None if self.turbo else _UNCOND)

    def velocity(self, heavy: _Heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        B, C, gh, gw = x.shape
        z = x.reshape(B, C, gh * gw).transpose(1, 2)
        t = torch.full((B,), 1.0 - sigma)
        if isinstance(cond, str):                               # unconditional DiT: image rows only, zero features
            pos, ind = packing(0, gh, gw)
            llm = torch.zeros(B, gh * gw, self.dit_cfg.llm_features_dim, device=self.device, dtype=self.dtype)
            v = heavy.uncond.forward(llm, z, t, pos, ind)
        else:
            n = cond.shape[1]
            pos, ind = packing(n, gh, gw)
            llm = torch.cat([cond.to(self.device, self.dtype),
                             torch.zeros(B, gh * gw, cond.shape[2], device=self.device, dtype=self.dtype)], dim=1)
            zz = torch.cat([torch.zeros(B, n, C, device=x.device, dtype=x.dtype), z], dim=1)
            v = heavy.dit.forward(llm, zz, t, pos, ind)[:, n:]
        return -v.transpose(1, 2).reshape(B, C, gh, gw)

    def decode(self, heavy: _Heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        B, C, gh, gw = z.shape
        tok = z.to(self.device).float() * heavy.bn_std + heavy.bn_mean
        lat = tok.permute(0, 2, 3, 1).reshape(B, gh, gw, 2, 2, 32).permute(0, 5, 1, 3, 2, 4).reshape(B, 32, gh * 2, gw * 2)
        return self.decode_latent(heavy, lat, req)


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, IdeogramPipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random Ideogram-shaped snapshot (hash prompt features) with both DiTs and a turbo adapter."""
    from ..io.safetensors_io import save_file
    from .chroma import native_vae_to_diffusers

    root = Path(root)
    dit = IdeogramConfig(emb_dim=48, num_layers=2, num_heads=2, mlp_dim=96, adaln_dim=16, llm_features_dim=39,
                         mrope_section=(4, 4, 4))
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1, z_channels=32, scale_factor=1.0, shift_factor=0.0)
    for d, s in (("transformer", seed), ("unconditional_transformer", seed + 2)):
        (root / d).mkdir(parents=True, exist_ok=True)
        save_file(random_ideogram_weights(dit, s), root / d / "diffusion_pytorch_model.safetensors")
    (root / "vae").mkdir(exist_ok=True)
    g = torch.Generator().manual_seed(seed + 7)
    vae_sd = native_vae_to_diffusers(random_vae_weights(vae, seed + 1), len(vae.ch_mult))
    vae_sd["bn.running_mean"] = 0.1 * torch.randn(128, generator=g)
    vae_sd["bn.running_var"] = 0.5 + torch.rand(128, generator=g)
    save_file({k: v.float() for k, v in vae_sd.items()}, root / "vae" / "diffusion_pytorch_model.safetensors")
    r = 2
    save_file({"diffusion_model.layers.0.attention.qkv.lora_down.weight": 0.1 * torch.randn(r, 48, generator=g),
               "diffusion_model.layers.0.attention.qkv.lora_up.weight": 0.1 * torch.randn(144, r, generator=g),
               "diffusion_model.layers.1.feed_forward.w2.lora_A.weight": 0.1 * torch.randn(r, 96, generator=g),
               "diffusion_model.layers.1.feed_forward.w2.lora_B.weight": 0.1 * torch.randn(48, r, generator=g)},
              root / TURBO_LORA_FILE)
    d = {k: getattr(dit, k) for k in IdeogramConfig.__dataclass_fields__}
    d["mrope_section"] = list(dit.mrope_section)
    (root / "swb_config.json").write_text(json.dumps({
        "dit": d, "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks},
        "text": "hash"}))
    return root
