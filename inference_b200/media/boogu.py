"""Boogu-Image providers `boogu_image`, `boogu_image_turbo`, `boogu_image_edit` (and `cpu_*`) (parity:
candle-gen-boogu/src/{lib,pipeline,tokenizer,text_encoder,config}.rs).

* `boogu_image`: 50-step rectified flow over a statically shifted schedule (mu = 1.15), true classifier-free guidance
  4.0 whose negative is the EMPTY instruction under the "drop" system prompt (no user negative prompt); a REFERENCE
  image with a strength starts the run part-way from the encoded reference (image -> image).
* `boogu_image_turbo`: the same network with distilled weights, 4 steps, no guidance. Its native loop is the
  distillation's own: predict the clean sample from the current one, then re-noise it to the next level with fresh seeded
  noise. Asking for a sampler / scheduler (or image -> image) runs the ordinary flow sampler on the same levels.
* `boogu_image_edit`: up to five reference images. Each is encoded by the autoencoder into the DiT's reference token
  sequence AND read by the Qwen3-VL vision tower, whose tokens replace the image placeholders of the instruction (with
  DeepStack taps and three-axis positions), so the instruction states are image-grounded.

The instruction encoder is the Qwen3-VL-8B language tower under `mllm/` (final-norm states of every prompt token,
rendered as a ChatML system + user pair with a fixed system prompt per mode); latents are the FLUX.1 16-channel space.
The network takes t = 1 - sigma and predicts the velocity towards the data, so the framework's velocity is its negative."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..contracts.gen_core.generator import ConditioningKind, GenerationRequest
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import ProgressDecoding, ProgressStep
from ..models.dit_boogu import BooguConfig, BooguDiT, random_boogu_weights
from ..models.vae import OracleVaeDecoder, VaeConfig
from .family import FamilyPipeline, HashPromptEncoder, Variant, family_registrations, rgb8_image
from .reference import encode_reference_image, init_time_step, reference_of
from .seed import STEP_RNG_SALT, U64, default_seed, for_each_image_seed, seeded_noise_nchw

SYSTEM_PROMPT_T2I = ("You are a helpful assistant that generates high-quality images based on user instructions. "
                     "The instructions are as follows.")
SYSTEM_PROMPT_DROP = ("Describe the key features of the input image (color, shape, size, texture, objects, background), then "
                      "explain how the user's text instruction should alter or modify the image. Generate a new image that meets "
                      "the user's requirements while maintaining consistency with the original input where appropriate.")
MAX_TEXT_TOKENS, MAX_EDIT_TOKENS, MAX_EDIT_REFERENCES, IMAGE_TOKEN_ID = 1280, 8192, 5, 151655
SEQ_LEN, BASE_SHIFT, MAX_SHIFT, TURBO_SIGMA = 4096.0, 0.5, 1.15, 0.001
TURBO_SAMPLERS = ["lcm", "euler_ancestral", "dpmpp_sde"]

BASE = Variant("boogu_image", "boogu", 50, 4.0, conditioning=(ConditioningKind.REFERENCE,), extra={"no_negative": True})
TURBO = Variant("boogu_image_turbo", "boogu", 4, None, conditioning=(ConditioningKind.REFERENCE,),
                extra={"samplers": TURBO_SAMPLERS})
EDIT = Variant("boogu_image_edit", "boogu", 50, 4.0, conditioning=(ConditioningKind.REFERENCE, ConditioningKind.MULTI_REFERENCE),
               extra={"no_negative": True})
VARIANTS = [BASE, TURBO, EDIT]


def render_chat(system: str, user: str, image_tokens: list[int] | None = None) -> str:
    """ChatML system + user turn, no generation prompt; one vision block per reference in front of the user text."""
    vis = "".join("<|vision_start|>" + "<|image_pad|>" * n + "<|vision_end|>" for n in (image_tokens or []))
    return f"<|im_start|>system\n{system}<|im_end|>\n<|im_start|>user\n{vis}{user}<|im_end|>\n"


def lin_mu(seq_len: float = SEQ_LEN) -> float:
    m = (MAX_SHIFT - BASE_SHIFT) / (4096.0 - 256.0)
    return m * seq_len + BASE_SHIFT - m * 256.0


def base_sigmas(steps: int) -> list[float]:
    """sigma = 1 - t over t_i = shift(i / steps), a final 0: the exponential time shift with mu fixed at 1.15."""
    mu = lin_mu()

    def shift(t: float) -> float:
        t1 = min(max(1.0 - t, 1e-8), 1.0 - 1e-8)
        return 1.0 - math.exp(mu) / (math.exp(mu) + (1.0 / t1 - 1.0))

    return [1.0 - shift(i / steps) for i in range(steps)] + [0.0]


def dmd_levels(steps: int, start: float = TURBO_SIGMA) -> list[float]:
    """Data fractions t_k the distilled student is conditioned on: linear from `start` towards 1 (exclusive)."""
    return [start + (1.0 - start) * k / steps for k in range(steps)]


def turbo_sigmas(steps: int) -> list[float]:
    return [1.0 - c for c in dmd_levels(steps)] + [0.0]


def edit_references(req: GenerationRequest) -> list[Image]:
    refs: list[Image] = []
    for c in req.conditioning:
        if c.kind is ConditioningKind.REFERENCE and c.image is not None:
            refs.append(c.image)
        elif c.kind is ConditioningKind.MULTI_REFERENCE:
            refs.extend(c.images)
    if not refs:
        raise InferenceError("boogu_image_edit: an instruction edit requires at least one source reference image")
    if len(refs) > MAX_EDIT_REFERENCES:
        raise InferenceError(f"boogu_image_edit: at most {MAX_EDIT_REFERENCES} reference images are supported (got {len(refs)})")
    return refs


class BooguInstructionEncoder:
    """Final-norm states of every token of the rendered chat; with images, the vision tower's tokens replace the
    placeholder embeddings, DeepStack taps are added after the first decoder layers and positions are three-axis."""

    def __init__(self, lm, tokenizer, weights=None, vision_cfg=None, device="cpu", image_token_id: int = IMAGE_TOKEN_ID):
        self.lm, self.tok, self.device, self.image_token_id = lm, tokenizer, device, image_token_id
        self.image_limits: dict = {}          # min_pixels / max_pixels of the vision preprocessor, when not its defaults
        self._weights, self._vision_cfg, self._vision, self._oracle = weights, vision_cfg, None, None

    def _ids(self, text: str, cap: int, what: str) -> list[int]:
        ids = self.tok.encode(text, add_special_tokens=False).ids
        if not ids or len(ids) > cap:
            raise InferenceError(f"boogu: the {what} renders to {len(ids)} tokens (supported: 1..={cap})")
        return ids

    def encode(self, prompt: str) -> torch.Tensor:
        return self.lm.encode(self._ids(render_chat(SYSTEM_PROMPT_T2I, prompt), MAX_TEXT_TOKENS, "prompt"))

    def encode_negative(self) -> torch.Tensor:
        return self.lm.encode(self._ids(render_chat(SYSTEM_PROMPT_DROP, ""), MAX_TEXT_TOKENS, "negative"))

    def encode_edit(self, instruction: str, images: list[Image]) -> torch.Tensor:
        from ..models.oracle import OracleLlama, canonical_weights
        from ..models.qwen3_vl import Qwen3VlVisionTower, image_to_patches, mrope_positions

        if self._weights is None or self._vision_cfg is None:
            raise LoadError("boogu_image_edit: the snapshot's mllm/ has no vision tower (model.visual.*)")
        if self._vision is None:
            self._vision = Qwen3VlVisionTower(self._vision_cfg, self._weights, self.device, torch.float32)
            lmw = {"model." + k[len("model.language_model."):]: v for k, v in self._weights.items()
                   if k.startswith("model.language_model.")}
            self._oracle = OracleLlama(self.lm.cfg, canonical_weights(lmw, self.lm.cfg), torch.float32, self.device)
        embeds, taps, grids = [], [], []
        for im in images:
            rgb = torch.frombuffer(bytearray(im.pixels), dtype=torch.uint8).view(im.height, im.width, 3)
            patches, grid = image_to_patches(rgb, self._vision_cfg, **self.image_limits)
            e, d = self._vision.forward(patches, [grid])
            embeds.append(e)
            taps.append(d)
            grids.append(grid)
        ids = self._ids(render_chat(SYSTEM_PROMPT_DROP, instruction, [e.shape[0] for e in embeds]), MAX_EDIT_TOKENS,
                        "image-grounded instruction")
        t = torch.tensor([ids], dtype=torch.int64, device=self.device)
        x = self._oracle.embed(t).clone()
        rows = (t[0] == self.image_token_id).nonzero()[:, 0]
        x[0, rows] = torch.cat(embeds, 0).to(x.dtype)
        stack = [torch.cat([d[i] for d in taps], 0) for i in range(len(taps[0]))]
        pos, _ = mrope_positions(ids, grids, self.image_token_id, self._vision_cfg.spatial_merge_size)
        h = self._oracle.hidden_states(None, None, embeds=x, mrope_positions=pos, deepstack=(rows, stack))
        return self._oracle._norm(h, "model.norm.weight")


@dataclass
class _Heavy:
    dit: Any
    vae: Any


class BooguPipeline(FamilyPipeline):
    def __init__(self, variant, root, backend, device):
        super().__init__(variant, root, backend, device)
        self.dit_cfg, self.vae_cfg = BooguConfig(), VaeConfig()
        if "dit" in self.raw:
            self.dit_cfg = BooguConfig.from_json(self.raw["dit"])
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = BooguConfig.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        if "vae" in self.raw:
            v = dict(self.raw["vae"])
            v["ch_mult"] = tuple(v.get("ch_mult", self.vae_cfg.ch_mult))
            self.vae_cfg = VaeConfig(**v)

    # ---- components ---------------------------------------------------------------------------------------------------
    def load_text(self):
        if self.text_kind == "hash":
            h = HashPromptEncoder(self.dit_cfg.text_dim, self.device, self.dtype)

            class _Hash:
                def encode(self, prompt: str):
                    return h.encode(render_chat(SYSTEM_PROMPT_T2I, prompt)).txt

                def encode_negative(self):
                    return h.encode(render_chat(SYSTEM_PROMPT_DROP, "")).txt

                def encode_edit(self, instruction: str, images):
                    tag = "".join(f"[{im.width}x{im.height}:{sum(im.pixels[:64])}]" for im in images)
                    return h.encode(render_chat(SYSTEM_PROMPT_DROP, tag + instruction)).txt

            return _Hash()
        import tokenizers

        from ..io.safetensors_io import load_dir
        from ..models.qwen3_vl import Qwen3VlVisionConfig, language_model_config
        from ..models.text_encoders import CausalLmTextEncoder

        mllm = self.root / "mllm"
        if not (mllm / "config.json").is_file() or not (mllm / "tokenizer.json").is_file():
            raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks mllm/config.json or mllm/tokenizer.json")
        cj = json.loads((mllm / "config.json").read_text())
        cfg = language_model_config(cj)
        raw = load_dir(mllm)
        lmw = {"model." + k[len("model.language_model."):]: v for k, v in raw.items() if k.startswith("model.language_model.")}
        lm = CausalLmTextEncoder(cfg, lmw, self.device, skip_last=0, final_norm=True)
        has_vision = any(k.startswith("model.visual.") for k in raw) and "vision_config" in cj
        keep = raw if (has_vision and self.variant is EDIT) else None
        vcfg = Qwen3VlVisionConfig.from_json(cj["vision_config"]) if has_vision else None
        return BooguInstructionEncoder(lm, tokenizers.Tokenizer.from_file(str(mllm / "tokenizer.json")), keep, vcfg, self.device,
                                       int(cj.get("image_token_id", IMAGE_TOKEN_ID)))

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir
        from ..models.vae import random_vae_weights
        from .chroma import convert_diffusers_vae_decoder

        if self.random_init is not None:
            seed = int(self.random_init)
            dit_w, vae_w = random_boogu_weights(self.dit_cfg, seed), random_vae_weights(self.vae_cfg, seed + 1)
        else:
            for d in ("transformer", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {d}/")
            dit_w = load_dir(self.root / "transformer")
            vae_w = convert_diffusers_vae_decoder(load_dir(self.root / "vae"), len(self.vae_cfg.ch_mult))
        if self.backend == "b200":
            from ..models.vae import VaeDecoderGpu

            vae = VaeDecoderGpu(self.vae_cfg, self.device)
            vae = vae.init_random(int(self.random_init) + 1) if self.random_init is not None else vae.load_state_dict(vae_w)
        else:
            vae = OracleVaeDecoder(self.vae_cfg, vae_w, device=self.device)
        return _Heavy(BooguDiT(self.dit_cfg, dit_w, self.dtype, self.device), vae)

    def reference_latent(self, image: Image, width: int, height: int) -> torch.Tensor:
        from ..io.safetensors_io import load_dir
        from .chroma import convert_diffusers_vae_encoder

        return encode_reference_image(self.vae_cfg, convert_diffusers_vae_encoder(load_dir(self.root / "vae")), image, width,
                                      height, self.device, self.variant.id)

    # ---- program hooks ------------------------------------------------------------------------------------------------
    def validate(self, req: GenerationRequest) -> None:
        if not req.prompt.strip():
            raise InferenceError(f"{self.variant.id}: prompt must not be empty")
        if self.variant is EDIT:
            for i, r in enumerate(edit_references(req)):
                if r.width % self.variant.size_multiple or r.height % self.variant.size_multiple:
                    raise InferenceError(f"boogu_image_edit: reference {i} dims must be multiples of "
                                         f"{self.variant.size_multiple} (got {r.width}x{r.height})")
        else:
            reference_of(req, self.variant.id)

    def encode(self, text, req: GenerationRequest):
        g = self.guidance(req)
        neg = text.encode_negative() if self.cfg_active(g) else None
        if self.variant is EDIT:
            return text.encode_edit(req.prompt, edit_references(req)), neg
        return text.encode(req.prompt), neg

    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        return turbo_sigmas(steps) if self.variant is TURBO else base_sigmas(steps)

    def scheduler_mu(self, req: GenerationRequest) -> float:
        if req.scheduler_shift is not None:
            return req.scheduler_shift
        return 0.0 if self.variant is TURBO else lin_mu()

    def combine(self, cond_v, uncond_v, guidance):
        return cond_v + (cond_v - uncond_v) * (guidance - 1.0)

    def velocity(self, heavy: _Heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        t = torch.full((1,), 1.0 - float(sigma), device=self.device)
        return -heavy.dit.forward(x, t, cond, self._refs)

    def decode(self, heavy: _Heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        if self.backend == "b200":
            host = heavy.vae.decode_rgb8(z.to(self.device))[0].cpu()
            return [Image(width=req.width, height=req.height, pixels=host.contiguous().numpy().tobytes())]
        return [rgb8_image(heavy.vae.decode(z)[0], req.width, req.height)]

    _refs: tuple = ()
    _start: tuple | None = None

    def sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        s = super().sigmas(steps, req)
        return s[self._start[0]:] if self._start is not None else s

    def initial_latent(self, seed: int, req: GenerationRequest) -> torch.Tensor:
        noise = super().initial_latent(seed, req)
        if self._start is None:
            return noise
        _, clean, sigma0 = self._start
        return clean.cpu().float() * (1.0 - sigma0) + noise * sigma0

    def render(self, heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        v = self.variant
        steps = req.steps or v.default_steps
        self._refs, self._start = (), None
        if v is EDIT:
            self._refs = tuple(self.reference_latent(r, r.width, r.height).to(self.device) for r in edit_references(req))
        else:
            ref = reference_of(req, v.id)
            strength = None if ref is None else (ref[1] if ref[1] is not None else req.strength)
            if ref is not None and init_time_step(steps, strength) > 0:
                full = super().sigmas(steps, req)
                start = min(init_time_step(steps, strength), len(full) - 2)
                self._start = (start, self.reference_latent(ref[0], req.width, req.height), full[start])
        try:
            if v is TURBO and self._start is None and req.sampler is None and req.scheduler is None:
                return self._render_dmd(heavy, cond[0], req, steps, on_progress)
            return super().render(heavy, cond, req, on_progress)
        finally:
            self._refs, self._start = (), None

    def _render_dmd(self, heavy, cond, req, steps: int, on_progress) -> list[Image]:
        levels = dmd_levels(steps)
        c, h, w = self.latent_shape(req)
        base_seed = req.seed if req.seed is not None else default_seed()

        def one(seed: int):
            x = seeded_noise_nchw(seed, c, h, w).to(self.device).float()
            for i, t in enumerate(levels):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{self.variant.id}: cancelled at step {i}")
                pred = heavy.dit.forward(x.to(self.dtype), torch.full((1,), t, device=self.device), cond).float()
                x = x + pred * (1.0 - t)                                    # the predicted clean sample
                if i + 1 < steps:
                    fresh = seeded_noise_nchw((seed + STEP_RNG_SALT + i + 1) & U64, c, h, w).to(self.device).float()
                    x = fresh * (1.0 - levels[i + 1]) + x * levels[i + 1]
                on_progress(ProgressStep(i + 1, steps))
            on_progress(ProgressDecoding())
            return self.decode(heavy, x, req)

        return [img for imgs in for_each_image_seed(base_seed, req.count, one) for img in imgs]


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, BooguPipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random Boogu-shaped snapshot: 1 double + 2 single + 1 refiner layers of width 96 (4 / 2 heads of 24), the
    weight-free prompt encoder, a small FLUX-layout autoencoder with its encoder."""
    from ..io.safetensors_io import save_file
    from ..models.vae import random_vae_encoder_weights, random_vae_weights
    from .chroma import native_vae_to_diffusers
    from .z_image import native_vae_encoder_to_diffusers

    root = Path(root)
    cfg = dict(hidden_size=96, num_layers=3, num_double_stream_layers=1, num_refiner_layers=1, num_attention_heads=4,
               num_kv_heads=2, axes_dim_rope=[8, 8, 8], text_dim=32, multiple_of=32)
    dit = BooguConfig.from_json(cfg)
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file(random_boogu_weights(dit, seed), root / "transformer" / "diffusion_pytorch_model.safetensors")
    sd = native_vae_to_diffusers(random_vae_weights(vae, seed + 1), len(vae.ch_mult))
    sd.update(native_vae_encoder_to_diffusers(random_vae_encoder_weights(vae, seed + 3)))
    save_file({k: v.bfloat16() for k, v in sd.items()}, root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": cfg, "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks}, "text": "hash"}))
    return root
