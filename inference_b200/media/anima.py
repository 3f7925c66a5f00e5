"""Anima text-to-image providers `anima_base`, `anima_aesthetic`, `anima_turbo` (and `cpu_*` on the fp32 oracle backend)
(parity: candle-gen-anima/src/lib.rs, pipeline.rs, loader.rs, tokenizer.rs, adapters.rs).

One architecture, three checkpoints. The prompt is tokenised twice: Qwen3-0.6B states of the Qwen tokens (masked) are
the source, T5 token ids the target of the bundled text conditioner, whose 512-row output the Cosmos DiT
cross-attends. base / aesthetic: 30 steps, true classifier-free guidance 4.5 (negative prompt default ""); turbo: 10
steps, one forward per step. Sigmas are linspace(1, 1/N) through a static shift of 3, the default solver is `er_sde`,
and the network sees sigma itself. 16-channel latents at 1/8 resolution decode through the Qwen-Image autoencoder.
LoRA and LoKr files are folded into the DiT and conditioner weights at load, with strict routing.

Snapshot layout: `diffusion_models/anima-<variant>-v1.0.safetensors` (DiT + `llm_adapter.*` under one root prefix),
`text_encoders/qwen_3_06b_base.safetensors`, `vae/qwen_image_vae.safetensors`, `tokenizers/qwen.json` and
`tokenizers/t5.json`; the same tree under `split_files/` is accepted."""
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
from ..models.dit_anima import (AnimaTextConditioner, ConditionerConfig, CosmosConfig, CosmosDiT, anima_sigmas, convert_vae_key,
                                detect_dit_prefix, random_anima_weights)
from ..models.vae_qwen import QwenVaeConfig, QwenVaeDecoder, random_qwen_vae_weights
from .family import FamilyPipeline, HashPromptEncoder, Variant, family_registrations, fold_adapters, rgb8_image
from .seed import seeded_noise_nchw

MAX_LEN, DEFAULT_SAMPLER, SIGMA_SHIFT = 512, "er_sde", 3.0
TEXT_ENCODER_FILE, VAE_FILE = "text_encoders/qwen_3_06b_base.safetensors", "vae/qwen_image_vae.safetensors"
QWEN3_06B = dict(vocab_size=151936, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                 head_dim=128, intermediate_size=3072, rope_theta=1_000_000.0, rms_norm_eps=1e-6, model_type="qwen3",
                 tie_word_embeddings=True)


def _variant(name: str, steps: int, guidance: float | None) -> Variant:
    return Variant(f"anima_{name}", "anima", steps, guidance, size_multiple=16, min_size=512, max_size=1536,
                   supports_lora=True, supports_lokr=True, extra={"file": f"anima-{name}-v1.0.safetensors"})


VARIANTS = [_variant("base", 30, 4.5), _variant("aesthetic", 30, 4.5), _variant("turbo", 10, None)]


class AnimaPromptEncoder:
    def __init__(self, lm, qwen_tok, t5_tok, device):
        self.lm, self.qwen, self.t5, self.device = lm, qwen_tok, t5_tok, device

    def encode(self, prompt: str):
        """-> (masked Qwen3 states [1, S, 1024], T5 ids [1, St])."""
        q = self.qwen.encode(prompt, add_special_tokens=False).ids[:MAX_LEN]
        t = self.t5.encode(prompt, add_special_tokens=True).ids[:MAX_LEN]
        if not q or not t:
            raise InferenceError("anima: the prompt tokenised to nothing")
        return self.lm.encode(q), torch.tensor([t], dtype=torch.int64)


@dataclass
class _Text:
    encoder: Any
    conditioner: AnimaTextConditioner

    def encode(self, prompt: str) -> torch.Tensor:
        src, ids = self.encoder.encode(prompt)
        return self.conditioner.forward(src, ids)


@dataclass
class _Heavy:
    dit: CosmosDiT
    vae: QwenVaeDecoder


class AnimaPipeline(FamilyPipeline):
    latent_channels = 16
    latent_downscale = 8

    def __init__(self, variant, root, backend, device):
        super().__init__(variant, root, backend, device)
        if not (self.root / "diffusion_models").is_dir() and (self.root / "split_files" / "diffusion_models").is_dir():
            self.root = self.root / "split_files"
        self.dit_cfg = CosmosConfig.from_json(self.raw["dit"]) if "dit" in self.raw else CosmosConfig()
        self.cond_cfg = ConditionerConfig.from_json(self.raw["conditioner"]) if "conditioner" in self.raw else ConditionerConfig()
        v = dict(self.raw.get("vae", {}))
        if "dim_mult" in v:
            v["dim_mult"] = tuple(v["dim_mult"])
        self.vae_cfg = QwenVaeConfig(**v)
        self.latent_channels = self.dit_cfg.in_channels
        self._weights = None

    def _dit_weights(self) -> dict[str, torch.Tensor]:
        """The checkpoint with its root prefix stripped and adapters folded (shared by the text and heavy stages)."""
        if self._weights is None:
            from ..io.safetensors_io import load_file

            if self.random_init is not None:
                w = random_anima_weights(self.dit_cfg, self.cond_cfg, int(self.random_init), 0.02)
            else:
                path = self.root / "diffusion_models" / self.variant.extra["file"]
                if not path.is_file():
                    raise LoadError(f"{self.variant.id}: {path} not found")
                raw = load_file(path)
                try:
                    pre = detect_dit_prefix(raw) + "."
                except ValueError as e:
                    raise LoadError(f"{self.variant.id}: {e}") from None
                w = {k[len(pre):]: v for k, v in raw.items() if k.startswith(pre)}
            self._weights = fold_adapters(w, self.adapters, self.variant.id)
        return self._weights

    def load_text(self):
        cond = AnimaTextConditioner(self.cond_cfg, self._dit_weights(), self.dtype, self.device)
        if self.text_kind == "hash":
            h = HashPromptEncoder(self.cond_cfg.source_dim, self.device, self.dtype)
            vocab = self.cond_cfg.target_vocab_size

            class _Hash:
                def encode(self, prompt: str):
                    b = prompt.encode("utf-8") or b"\0"
                    return h.encode(prompt).txt, torch.tensor([[(x * 7 + i) % vocab for i, x in enumerate(b)][:MAX_LEN] + [1]])
            return _Text(_Hash(), cond)
        import tokenizers

        from ..io.safetensors_io import load_file
        from ..models.config import ModelConfig
        from ..models.text_encoders import CausalLmTextEncoder

        te = self.root / TEXT_ENCODER_FILE
        qt, tt = self.root / "tokenizers" / "qwen.json", self.root / "tokenizers" / "t5.json"
        for f in (te, qt, tt):
            if not f.is_file():
                raise LoadError(f"{self.variant.id}: {f} not found")
        cfg = ModelConfig.from_json({**QWEN3_06B, **self.raw.get("text_encoder", {})})
        w = {(k if k.startswith("model.") else "model." + k): v for k, v in load_file(te).items()}
        lm = CausalLmTextEncoder(cfg, w, self.device, skip_last=0, final_norm=True)
        return _Text(AnimaPromptEncoder(lm, tokenizers.Tokenizer.from_file(str(qt)), tokenizers.Tokenizer.from_file(str(tt)),
                                        self.device), cond)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_file

        if self.random_init is not None:
            vae_w = random_qwen_vae_weights(self.vae_cfg, int(self.random_init) + 1)
        else:
            vf = self.root / VAE_FILE
            if not vf.is_file():
                raise LoadError(f"{self.variant.id}: {vf} not found")
            vae_w = {convert_vae_key(k): v for k, v in load_file(vf).items()}
        heavy = _Heavy(CosmosDiT(self.dit_cfg, self._dit_weights(), self.dtype, self.device),
                       QwenVaeDecoder(self.vae_cfg, vae_w, self.dtype, self.device))
        self._weights = None
        return heavy

    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        return anima_sigmas(steps, SIGMA_SHIFT)

    def scheduler_mu(self, req):
        import math

        return req.scheduler_shift if req.scheduler_shift is not None else math.log(SIGMA_SHIFT)

    def validate(self, req: GenerationRequest) -> None:
        mh, mw = self.dit_cfg.max_size[1] * self.dit_cfg.patch_size[1] * 8, self.dit_cfg.max_size[2] * self.dit_cfg.patch_size[2] * 8
        if req.height > mh or req.width > mw:
            raise InferenceError(f"{self.variant.id}: {req.width}x{req.height} exceeds the rotary tables' {mw}x{mh}")

    def render(self, heavy, cond, req: GenerationRequest, on_progress):
        if req.sampler is None:
            import dataclasses

            req = dataclasses.replace(req, sampler=DEFAULT_SAMPLER)
        return super().render(heavy, cond, req, on_progress)

    def initial_latent(self, seed: int, req: GenerationRequest) -> torch.Tensor:
        C, h, w = self.latent_shape(req)
        return seeded_noise_nchw(seed, C, h, w).reshape(1, C, 1, h, w)

    def velocity(self, heavy: _Heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        return heavy.dit.forward(x, torch.full((x.shape[0],), sigma), cond)

    def decode(self, heavy: _Heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        return [rgb8_image(heavy.vae.decode(z[:, :, 0].to(self.device, self.dtype))[0], req.width, req.height)]


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, AnimaPipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0, prefix: str = "net") -> Path:
    """A tiny random Anima-shaped snapshot (hash prompt features) holding all three checkpoints."""
    from ..io.safetensors_io import save_file

    root = Path(root)
    dit = CosmosConfig(num_attention_heads=2, attention_head_dim=12, num_layers=2, text_embed_dim=16, adaln_lora_dim=8,
                       in_channels=16, out_channels=16, max_size=(4, 96, 96))
    cond = ConditionerConfig(source_dim=20, target_dim=16, model_dim=16, num_layers=2, num_attention_heads=2,
                             target_vocab_size=64, min_sequence_length=24)
    vae = QwenVaeConfig(base_dim=16, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    (root / "diffusion_models").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    for i, v in enumerate(VARIANTS):
        w = random_anima_weights(dit, cond, seed + i)
        save_file({f"{prefix}.{k}": t for k, t in w.items()}, root / "diffusion_models" / v.extra["file"])
    save_file(random_qwen_vae_weights(vae, seed + 9), root / VAE_FILE)
    jd = {k: (list(x) if isinstance(x := getattr(dit, k), tuple) else x) for k in CosmosConfig.__dataclass_fields__}
    jc = {k: getattr(cond, k) for k in ConditionerConfig.__dataclass_fields__}
    (root / "swb_config.json").write_text(json.dumps({
        "dit": jd, "conditioner": jc, "text": "hash",
        "vae": {"base_dim": vae.base_dim, "dim_mult": list(vae.dim_mult), "num_res_blocks": vae.num_res_blocks}}))
    return root
