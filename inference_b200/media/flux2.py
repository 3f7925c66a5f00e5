"""FLUX.2 text-to-image providers `flux2_klein_9b` and `flux2_dev` (and `cpu_*` on the fp32 oracle backend)
(parity: candle-gen-flux2/src/lib.rs, pipeline.rs, text_encoder.rs, vae.rs).

klein: Qwen3 hidden states after layers 9 / 18 / 27 concatenated per token (12288 wide), 4 flow-match Euler steps,
guidance 1.0 = one forward per step; a guidance above 1 adds a negative-prompt pass (default negative prompt " ")
blended as v_neg + g (v - v_neg). dev: Mistral layers 10 / 20 / 30 (15360 wide), ~28 steps, the guidance scale
(default 4) is an input of the network, no negative prompt. Prompts are right-padded to 512 tokens; padding is masked
as attention keys inside the text encoder and the DiT attends all 512 rows. The sigma table is 1 -> 1 / steps through
an exponential shift whose mu is an empirical function of image token count and step count; the network sees
sigma * 1000. Latents are 32-channel at 1/8 resolution, packed 2 x 2 into 128-channel tokens in a space normalised by
the autoencoder's batch-norm statistics.

Snapshot layout (diffusers): `transformer/`, `text_encoder/` + `tokenizer/tokenizer.json`, `vae/`."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
import torch.nn.functional as F

from ..contracts.errors import InferenceError, LoadError
from ..contracts.gen_core.generator import GenerationRequest
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..models.dit_flux2 import Flux2Config, Flux2DiT, grid_ids, random_flux2_weights, text_ids, vae_unpatchify
from ..models.vae import OracleVaeDecoder, VaeConfig, random_vae_weights
from .family import FamilyPipeline, HashPromptEncoder, Variant, family_registrations, rgb8_image

MAX_SEQUENCE = 512
VARIANTS = [
    Variant("flux2_klein_9b", "flux2", 4, 1.0, size_multiple=16,
            extra={"config": "klein_9b", "te_layers": (9, 18, 27), "template": "qwen_instruct_no_think"}),
    Variant("flux2_dev", "flux2", 28, 4.0, size_multiple=16, embedded_guidance=True,
            extra={"config": "dev", "te_layers": (10, 20, 30), "template": "flux2_dev_mistral"}),
]


def compute_mu(seq_len: int, num_steps: int) -> float:
    """Empirical shift: linear in the token count above 4300 tokens, below it interpolated in the step count between the
    10-step and the 200-step fits."""
    a1, b1, a2, b2 = 8.73809524e-5, 1.89833333, 0.00016927, 0.45666666
    if seq_len > 4300:
        return a2 * seq_len + b2
    m200, m10 = a2 * seq_len + b2, a1 * seq_len + b1
    a = (m200 - m10) / 190.0
    return a * num_steps + (m200 - 200.0 * a)


def build_sigmas(num_steps: int, mu: float) -> list[float]:
    e = math.exp(mu)
    out = []
    for i in range(num_steps):
        t = 1.0 if num_steps == 1 else 1.0 + (1.0 / num_steps - 1.0) * i / (num_steps - 1)
        out.append(e / (e + (1.0 / t - 1.0)))
    return out + [0.0]


class Flux2PromptEncoder:
    """Chat-templated prompt, right-padded to 512 tokens, through a decoder LM whose three tapped layers are
    concatenated on the feature axis. Padding rows are computed with padding masked as keys (a causal mask over the
    real tokens only), as the reference's host-built mask does."""

    def __init__(self, lm, tokenizer, layers: tuple[int, ...], pad_id: int, max_len: int = MAX_SEQUENCE):
        self.lm, self.tok, self.layers, self.pad_id, self.max_len = lm, tokenizer, layers, pad_id, max_len

    def encode(self, prompt: str) -> torch.Tensor:
        ids = self.tok.tokenize(prompt).ids[: self.max_len]
        n = len(ids)
        if n == 0:
            raise InferenceError("flux2: the prompt tokenised to nothing")
        full = ids + [self.pad_id] * (self.max_len - n)
        S = len(full)
        j = torch.arange(S)
        allowed = (j[None, :] <= j[:, None]) & (j[None, :] < n)
        allowed |= torch.eye(S, dtype=torch.bool) & (j[None, :] >= n)     # a padding row keeps itself (no empty rows)
        mask = torch.zeros(S, S).masked_fill(~allowed, float("-inf"))[None, None]
        t = torch.tensor([full], dtype=torch.int64)
        outs = [self.lm.hidden_states(t, None, num_layers=i, additive_mask=mask.to(self.lm.device, self.lm.dtype))
                for i in self.layers]
        return torch.cat(outs, dim=-1)


@dataclass
class _Heavy:
    dit: Flux2DiT
    vae: Any
    post_quant: tuple[torch.Tensor, torch.Tensor] | None
    bn_mean: torch.Tensor
    bn_std: torch.Tensor


class Flux2Pipeline(FamilyPipeline):
    latent_channels = 128
    latent_downscale = 16

    def __init__(self, variant, root, backend, device):
        super().__init__(variant, root, backend, device)
        self.dit_cfg = getattr(Flux2Config, variant.extra["config"])()
        self.vae_cfg = VaeConfig(z_channels=32, scale_factor=1.0, shift_factor=0.0)
        if "dit" in self.raw:
            self.dit_cfg = Flux2Config.from_json(self.raw["dit"])
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = Flux2Config.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        if "vae" in self.raw:
            v = dict(self.raw["vae"])
            if "ch_mult" in v:
                v["ch_mult"] = tuple(v["ch_mult"])
            self.vae_cfg = VaeConfig(**{"z_channels": 32, "scale_factor": 1.0, "shift_factor": 0.0, **v})
        self.max_len = int(self.raw.get("max_sequence_length", MAX_SEQUENCE))

    def load_text(self):
        if self.text_kind == "hash":
            h = HashPromptEncoder(self.dit_cfg.joint_attention_dim, self.device, self.dtype)
            n = self.max_len

            class _Fixed:
                def encode(self, prompt: str):
                    return h.encode(prompt, n).txt
            return _Fixed()
        from ..contracts.gen_core.tokenizer import PromptTemplate, TextTokenizer, TokenizerConfig
        from ..io.safetensors_io import load_dir
        from ..models.config import ModelConfig
        from ..models.oracle import OracleLlama

        te, tk = self.root / "text_encoder", self.root / "tokenizer" / "tokenizer.json"
        if not te.is_dir() or not tk.exists():
            raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks text_encoder/ or tokenizer/tokenizer.json")
        top = json.loads((te / "config.json").read_text())
        cfg = ModelConfig.from_json(top.get("text_config", top))
        w = {}
        for k, v in load_dir(te).items():
            w["model." + k[len("language_model.model."):] if k.startswith("language_model.model.") else k] = v
        tmpl = PromptTemplate.QWEN_INSTRUCT if "qwen" in self.variant.extra["template"] else PromptTemplate.NONE
        tok = TextTokenizer.from_file(tk, TokenizerConfig(max_length=self.max_len, chat_template=tmpl))
        lm = OracleLlama(cfg, w, self.dtype, self.device)
        pad = int(top.get("pad_token_id") or 0)
        return Flux2PromptEncoder(lm, tok, tuple(self.raw.get("te_layers", self.variant.extra["te_layers"])), pad, self.max_len)

    def load_vae(self):
        """(decoder, post-quant 1x1 conv or None, bn mean, bn std [1, 128, 1, 1]) of the FLUX.2 autoencoder."""
        from ..io.safetensors_io import load_dir
        from .chroma import convert_diffusers_vae_decoder

        if self.random_init is not None:
            vae_w, extra = random_vae_weights(self.vae_cfg, int(self.random_init) + 1), {}
        else:
            if not (self.root / "vae").is_dir():
                raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks vae/")
            raw_vae = load_dir(self.root / "vae")
            vae_w = convert_diffusers_vae_decoder(raw_vae, len(self.vae_cfg.ch_mult))
            extra = {k: v for k, v in raw_vae.items() if k.startswith(("post_quant_conv.", "bn."))}
        if self.backend == "b200":
            from ..models.vae import VaeDecoderGpu

            vae = VaeDecoderGpu(self.vae_cfg, self.device).load_state_dict(vae_w)
        else:
            vae = OracleVaeDecoder(self.vae_cfg, vae_w, device=self.device)
        C = 128
        mean = extra.get("bn.running_mean", torch.zeros(C)).float().view(1, C, 1, 1).to(self.device)
        std = torch.sqrt(extra.get("bn.running_var", torch.ones(C) - 1e-4).float() + 1e-4).view(1, C, 1, 1).to(self.device)
        pq = None
        if "post_quant_conv.weight" in extra:
            pq = (extra["post_quant_conv.weight"].float().to(self.device), extra["post_quant_conv.bias"].float().to(self.device))
        return vae, pq, mean, std

    def decode_latent(self, heavy, lat: torch.Tensor, req: GenerationRequest) -> list[Image]:
        """[1, 32, H/8, W/8] de-normalised latent -> RGB8."""
        if heavy.post_quant is not None:
            lat = F.conv2d(lat, heavy.post_quant[0], heavy.post_quant[1])
        if self.backend == "b200":
            u8 = heavy.vae.decode_rgb8(lat)[0].cpu()
            return [Image(width=req.width, height=req.height, pixels=u8.contiguous().numpy().tobytes())]
        return [rgb8_image(heavy.vae.decode(lat)[0], req.width, req.height)]

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir

        if self.random_init is not None:
            dit_w = random_flux2_weights(self.dit_cfg, int(self.random_init), 0.02, self.dtype, self.device)
        else:
            if not (self.root / "transformer").is_dir():
                raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks transformer/")
            dit_w = load_dir(self.root / "transformer")
        return _Heavy(Flux2DiT(self.dit_cfg, dit_w, self.dtype, self.device), *self.load_vae())

    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        return build_sigmas(steps, compute_mu((req.height // 16) * (req.width // 16), steps))

    def scheduler_mu(self, req):
        return req.scheduler_shift if req.scheduler_shift is not None else \
            compute_mu((req.height // 16) * (req.width // 16), req.steps or self.variant.default_steps)

    def encode(self, text, req: GenerationRequest):
        g = self.guidance(req)
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt if req.negative_prompt else " ") if self.cfg_active(g) else None
        self._embedded = torch.full((1,), float(g)) if self.variant.embedded_guidance else None
        return pos, neg

    def velocity(self, heavy: _Heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        B, C, h, w = x.shape
        tokens = x.reshape(B, C, h * w).transpose(1, 2)
        t = torch.full((B,), sigma * 1000.0, device=self.device)
        out = heavy.dit.forward(tokens, cond, grid_ids(h, w), text_ids(cond.shape[1]), t, self._embedded)
        return out.transpose(1, 2).reshape(B, C, h, w)

    def decode(self, heavy: _Heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        return self.decode_latent(heavy, vae_unpatchify(z.to(self.device).float() * heavy.bn_std + heavy.bn_mean), req)


def registrations(backend: str = "b200") -> list[Registration]:
    return family_registrations(VARIANTS, Flux2Pipeline, backend)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random FLUX.2-shaped snapshot (hash prompt encoder, 32 padded prompt rows) in the diffusers layout."""
    from ..io.safetensors_io import save_file
    from .chroma import native_vae_to_diffusers

    root = Path(root)
    dit = Flux2Config(num_double_layers=1, num_single_layers=2, num_heads=2, head_dim=32, joint_attention_dim=48,
                      axes_dim=(8, 8, 8, 8), guidance_embed=True)
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1, z_channels=32, scale_factor=1.0, shift_factor=0.0)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_flux2_weights(dit, seed).items()},
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    g = torch.Generator().manual_seed(seed + 7)
    vae_sd = native_vae_to_diffusers(random_vae_weights(vae, seed + 1), len(vae.ch_mult))
    vae_sd["post_quant_conv.weight"] = torch.eye(32).view(32, 32, 1, 1) + 0.05 * torch.randn(32, 32, 1, 1, generator=g)
    vae_sd["post_quant_conv.bias"] = 0.01 * torch.randn(32, generator=g)
    vae_sd["bn.running_mean"] = 0.1 * torch.randn(128, generator=g)
    vae_sd["bn.running_var"] = 0.5 + torch.rand(128, generator=g)
    save_file({k: v.float() for k, v in vae_sd.items()}, root / "vae" / "diffusion_pytorch_model.safetensors")
    d = {k: getattr(dit, k) for k in Flux2Config.__dataclass_fields__}
    d["axes_dim"] = list(dit.axes_dim)
    (root / "swb_config.json").write_text(json.dumps({
        "dit": d, "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks},
        "text": "hash", "max_sequence_length": 32}))
    return root
