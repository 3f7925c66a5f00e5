"""Krea 2 text-to-image providers `krea_2_turbo` and `krea_2_raw` (and `cpu_*` on the fp32 oracle backend)
(parity: candle-gen-krea/src/lib.rs, pipeline.rs, schedule.rs, tokenizer.rs, text_encoder.rs).

One architecture, two checkpoints. Turbo is guidance-distilled: 8 Euler steps over the exponential-shift table with
the fixed mu 1.15, no negative prompt. Raw is the undistilled base: 52 steps, mu interpolated from the image token
count, classifier-free guidance whenever the scale is > 0 with Krea's offset-by-one rule
v = v_cond + g (v_cond - v_uncond) (default 3.5). The prompt is wrapped in a fixed system template, run through the
Qwen3-VL language model, twelve of its hidden layers are stacked per token and the 34 template-prefix tokens are
dropped. The network is conditioned on sigma itself and returns the flow velocity; latents are 16-channel NCHW at
1/8 resolution, decoded by the Qwen-Image autoencoder.

Snapshot layout (diffusers): `transformer/`, `text_encoder/` + `tokenizer/tokenizer.json`, `vae/`, optional
`model_index.json` (`patch_size`, `text_encoder_select_layers`). `LoadSpec.quantize` = NVFP4 repacks the block
projections on the device (W4A16, or W4A4 with `swb_config.json: {"nvfp4_act": "w4a4"}`)."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ..contracts.errors import InferenceError, LoadError
from ..contracts.gen_core.generator import GenerationRequest
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..models.dit_krea import KreaConfig, KreaDiT, random_krea_weights
from ..models.vae_qwen import QwenVaeConfig, QwenVaeDecoder
from .family import (FamilyPipeline, HashPromptEncoder, Variant, family_registrations, load_vl_text_tower, merged_adapters,
                     rgb8_image)

TURBO_MU, TURBO_STEPS = 1.15, 8
RAW_STEPS, RAW_GUIDANCE = 52, 3.5
BASE_SEQ_LEN, MAX_SEQ_LEN, BASE_SHIFT, MAX_SHIFT = 256.0, 6400.0, 0.5, 1.15
MAX_TEXT_TOKENS = 1024
PREFIX = ("<|im_start|>system\nDescribe the image by detailing the color, shape, size, texture, quantity, text, spatial "
          "relationships of the objects and background:<|im_end|>\n<|im_start|>user\n")
SUFFIX = "<|im_end|>\n<|im_start|>assistant\n"
PREFIX_TOKENS = 34
SELECT_LAYERS = (2, 5, 8, 11, 14, 17, 20, 23, 26, 29, 32, 35)

VARIANTS = [
    Variant("krea_2_turbo", "krea", TURBO_STEPS, None, supports_lora=True, extra={"quants": True}),
    Variant("krea_2_raw", "krea", RAW_STEPS, RAW_GUIDANCE, supports_lora=True, extra={"quants": True}),
]


def dynamic_mu(seq_len: float) -> float:
    """Linear in the image token count between (256, 0.5) and (6400, 1.15)."""
    slope = (MAX_SHIFT - BASE_SHIFT) / (MAX_SEQ_LEN - BASE_SEQ_LEN)
    return slope * seq_len + (BASE_SHIFT - slope * BASE_SEQ_LEN)


def krea_sigmas(steps: int, mu: float) -> list[float]:
    """linspace(1, 0, steps + 1) through the exponential time shift e^mu / (e^mu + (1 / t - 1))."""
    n = max(1, steps)
    e = math.exp(mu)
    out = []
    for i in range(n + 1):
        t = 1.0 - i / n
        out.append(0.0 if t <= 0.0 else e / (e + (1.0 / t - 1.0)))
    return out


def krea_cfg_combine(v_cond: torch.Tensor, v_uncond: torch.Tensor, guidance: float) -> torch.Tensor:
    """Krea's rule is offset by one from the usual form: at guidance 1 the usual form returns v_cond (no guidance),
    this one already extrapolates (candle-gen-krea/src/pipeline.rs:1665-1680)."""
    return v_cond + (v_cond - v_uncond) * guidance


class KreaPromptEncoder:
    """Template + tokenizer + the language model's selected hidden layers, template prefix dropped."""

    def __init__(self, encoder, tokenizer, select: tuple[int, ...], prefix_tokens: int):
        self.encoder, self.tok, self.select, self.prefix_tokens = encoder, tokenizer, list(select), prefix_tokens

    def encode(self, prompt: str) -> torch.Tensor:
        ids = self.tok.encode(PREFIX + prompt + SUFFIX).ids[:MAX_TEXT_TOKENS]
        if len(ids) <= self.prefix_tokens:
            raise InferenceError(f"krea: prompt has {len(ids)} tokens but the {self.prefix_tokens} template-prefix "
                                 "tokens leave nothing")
        return self.encoder.encode_layers(ids, self.select)[:, self.prefix_tokens:]


@dataclass
class _Heavy:
    dit: KreaDiT
    vae: Any


class KreaPipeline(FamilyPipeline):
    pid_space = "qwenimage"            # the Qwen-Image autoencoder's latent space

    def __init__(self, variant, root, backend, device):
        super().__init__(variant, root, backend, device)
        self.dit_cfg, self.vae_cfg = KreaConfig(), QwenVaeConfig()
        self.select, self.prefix_tokens = SELECT_LAYERS, PREFIX_TOKENS
        if "dit" in self.raw:
            self.dit_cfg = KreaConfig.from_json(self.raw["dit"])
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = KreaConfig.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        if "vae" in self.raw:
            v = dict(self.raw["vae"])
            if "dim_mult" in v:
                v["dim_mult"] = tuple(v["dim_mult"])
            self.vae_cfg = QwenVaeConfig(**v)
        mi = self.root / "model_index.json"
        if mi.exists():
            try:
                m = json.loads(mi.read_text())
            except json.JSONDecodeError as e:          # a damaged manifest must not silently fall back to defaults
                raise LoadError(f"{variant.id}: model_index.json is not valid JSON: {e}")
            if "patch_size" in m:
                self.dit_cfg.patch_size = int(m["patch_size"])
            if "text_encoder_select_layers" in m:
                self.select = tuple(int(i) for i in m["text_encoder_select_layers"])
        if "select_layers" in self.raw:
            self.select = tuple(self.raw["select_layers"])
        if "prefix_tokens" in self.raw:
            self.prefix_tokens = int(self.raw["prefix_tokens"])
        if len(self.select) != self.dit_cfg.num_text_layers:
            raise LoadError(f"{variant.id}: {len(self.select)} selected encoder layers but the DiT fuses "
                            f"{self.dit_cfg.num_text_layers}")
        self.latent_channels = self.dit_cfg.latent_channels
        self.quantize = None

    # ---- components ------------------------------------------------------------------------------------------------
    def load_text(self):
        if self.text_kind == "hash":
            return HashPromptEncoder(self.dit_cfg.text_hidden_dim, self.device, self.dtype, layers=self.dit_cfg.num_text_layers)
        enc, tok = load_vl_text_tower(self.variant.id, self.root, self.device, max(self.select))
        return KreaPromptEncoder(enc, tok, self.select, self.prefix_tokens)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir
        from ..models.vae_qwen import random_qwen_vae_weights

        if self.random_init is not None:
            seed = int(self.random_init)
            dit_w = random_krea_weights(self.dit_cfg, seed, 0.02, self.dtype, self.device)
            vae_w = random_qwen_vae_weights(self.vae_cfg, seed + 1)
        else:
            for d in ("transformer", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {d}/")
            dit_w = merged_adapters(load_dir(self.root / "transformer"), self.adapters, self.variant.id)
            vae_w = load_dir(self.root / "vae")
        dit = KreaDiT(self.dit_cfg, dit_w, self.dtype, self.device)
        del dit_w
        if self.quantize is not None or self.raw.get("nvfp4_act"):
            if self.device.type != "cuda":
                raise LoadError(f"{self.variant.id}: NVFP4 loading needs the sm_100a backend")
            dit.quantize_nvfp4(self.raw.get("nvfp4_act", "w4a16"), int(self.raw.get("nvfp4_skip", 0)))
        return _Heavy(dit, QwenVaeDecoder(self.vae_cfg, vae_w, self.dtype, self.device))

    # ---- program hooks ---------------------------------------------------------------------------------------------
    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        if not self.variant.uses_cfg:
            return krea_sigmas(steps, TURBO_MU)
        p = self.dit_cfg.patch_size * self.latent_downscale
        return krea_sigmas(steps, dynamic_mu((req.height // p) * (req.width // p)))

    def scheduler_mu(self, req: GenerationRequest) -> float:
        if req.scheduler_shift is not None:
            return req.scheduler_shift
        if not self.variant.uses_cfg:
            return TURBO_MU
        p = self.dit_cfg.patch_size * self.latent_downscale
        return dynamic_mu((req.height // p) * (req.width // p))

    def cfg_active(self, guidance):                      # the reference runs the unconditional branch iff guidance > 0
        return self.variant.uses_cfg and guidance is not None and guidance > 0.0

    def combine(self, cond_v, uncond_v, guidance):
        return krea_cfg_combine(cond_v, uncond_v, guidance)

    def encode(self, text, req: GenerationRequest):
        def one(prompt: str):
            e = text.encode(prompt)
            return {"ctx": e.txt if hasattr(e, "txt") else e, "fused": None}

        g = self.guidance(req)
        return one(req.prompt), (one(req.negative_prompt or "") if self.cfg_active(g) else None)

    def velocity(self, heavy: _Heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        if cond["fused"] is None:                        # the text branch does not depend on the timestep
            cond["fused"] = heavy.dit.text_fusion(cond["ctx"])
        t = torch.full((1,), sigma, device=self.device)
        return heavy.dit.forward(x, t, None, fused_context=cond["fused"])

    def decode(self, heavy: _Heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        img = heavy.vae.decode(z.to(self.device, self.dtype))[0]
        return [rgb8_image(img, req.width, req.height)]


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, KreaPipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random Krea-shaped snapshot (hash prompt encoder) in the diffusers directory layout."""
    from ..io.safetensors_io import save_file
    from ..models.vae_qwen import random_qwen_vae_weights

    root = Path(root)
    dit = KreaConfig(num_attention_heads=2, num_kv_heads=1, attention_head_dim=32, num_layers=2, intermediate_size=96,
                     axes_dims_rope=(8, 12, 12), num_text_layers=3, num_layerwise_text_blocks=1,
                     num_refiner_text_blocks=1, text_hidden_dim=64, text_intermediate_size=96,
                     text_num_attention_heads=2, text_num_kv_heads=2)
    vae = QwenVaeConfig(base_dim=16, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_krea_weights(dit, seed).items()},
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    save_file({k: v.bfloat16() for k, v in random_qwen_vae_weights(vae, seed + 1).items()},
              root / "vae" / "diffusion_pytorch_model.safetensors")
    d = {k: getattr(dit, k) for k in KreaConfig.__dataclass_fields__}
    d["axes_dims_rope"] = list(dit.axes_dims_rope)
    (root / "swb_config.json").write_text(json.dumps({
        "dit": d, "vae": {"base_dim": vae.base_dim, "dim_mult": list(vae.dim_mult), "num_res_blocks": vae.num_res_blocks},
        "text": "hash", "select_layers": [1, 2, 3]}))
    return root
