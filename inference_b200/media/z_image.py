"""Z-Image text-to-image providers `z_image_turbo` and `z_image` (and `cpu_*` on the fp32 oracle)
(parity: candle-gen-z-image/src/lib.rs, base.rs, pipeline.rs, common.rs).

generate(): the prompt goes through the Qwen instruct chat template and a Qwen3 decoder whose second-to-last layer
is the caption; the DiT is conditioned on 1 - sigma and its output is negated to get the flow velocity. Turbo is
guidance-distilled (4 steps, a linear sigma ramp, no negative prompt); the base model runs classifier-free guidance
(default 4.0, 50 steps, sigma ramp shifted by 6) with the empty negative prompt rendered through the same template.
Latents are 16-channel NCHW at 1/8 resolution; the VAE is the FLUX autoencoder in diffusers key names.

Snapshot layout (diffusers): `transformer/`, `text_encoder/` (Qwen3) + `tokenizer/tokenizer.json`, `vae/`;
`swb_config.json` in the root overrides dimensions for synthetic snapshots."""
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
from ..contracts.gen_core.tokenizer import PromptTemplate, TextTokenizer, TokenizerConfig
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.dit_zimage import OracleZImageDiT, ZImageConfig
from ..models.vae import OracleVaeDecoder, VaeConfig
from .chroma import convert_diffusers_vae_decoder, convert_diffusers_vae_encoder, native_vae_to_diffusers
from .flux import SIZE_MULTIPLE
from .residency import Residency
from .reference import encode_reference_image, init_time_step, reference_of  # noqa: F401
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw

MAX_PROMPT_TOKENS = 512
TRAIN_TIMESTEPS = 1000


class ZImageVariant(enum.Enum):
    TURBO = "z_image_turbo"
    BASE = "z_image"

    @property
    def default_steps(self) -> int:
        return 4 if self is ZImageVariant.TURBO else 50

    @property
    def default_guidance(self) -> float | None:
        return None if self is ZImageVariant.TURBO else 4.0

    @property
    def schedule_shift(self) -> float:
        return 3.0 if self is ZImageVariant.TURBO else 6.0


def flow_match_sigmas(steps: int, shift: float, apply_shift: bool) -> list[float]:
    """The flow-match Euler table: `steps` values evenly spaced from 1 to the smallest training sigma (the shifted
    1 / 1000), then 0. Turbo integrates that ramp as it is (its conditioning is 1 - sigma of the same ramp); the base
    model passes it through the static shift `s * x / (1 + (s - 1) * x)`."""
    lo = shift * (1.0 / TRAIN_TIMESTEPS) / (1.0 + (shift - 1.0) / TRAIN_TIMESTEPS)
    n = max(1, steps)
    ramp = [1.0 if n == 1 else 1.0 + (lo - 1.0) * i / (n - 1) for i in range(n)]
    if apply_shift:
        ramp = [shift * s / (1.0 + (shift - 1.0) * s) for s in ramp]
    return ramp + [0.0]


def z_image_sigmas(variant: ZImageVariant, steps: int) -> list[float]:
    return flow_match_sigmas(steps, variant.schedule_shift, apply_shift=variant is ZImageVariant.BASE)


# ---- prompt encoding ---------------------------------------------------------------------------------------------------------
class QwenCaptionEncoder:
    def __init__(self, encoder, tokenizer: TextTokenizer):
        self.encoder, self.tok = encoder, tokenizer

    def encode(self, prompt: str) -> torch.Tensor:
        """[1, L, hidden]; the empty prompt still renders the template's role markers."""
        ids = self.tok.tokenize(prompt).ids if prompt else self.tok.encode_chat_ids("", True)[:MAX_PROMPT_TOKENS]
        if not ids:
            raise InferenceError("z-image: the prompt tokenised to nothing")
        return self.encoder.encode(ids)


class HashCaptionEncoder:
    """Weight-free stand-in (synthetic snapshots)."""

    def __init__(self, dim: int, device, dtype):
        from .text_encoders import HashTextEncoders

        self.h = HashTextEncoders(dim, 8, device, dtype)

    def encode(self, prompt: str) -> torch.Tensor:
        return self.h.encode(prompt, 8 + len(prompt.encode("utf-8"))).txt


@dataclass
class _Heavy:
    dit: Any
    vae: Any


class ZImagePipeline:
    def __init__(self, variant: ZImageVariant, root: Path, backend: str, device: torch.device):
        self.variant, self.root, self.backend, self.device = variant, Path(root), backend, device
        self.dit_cfg, self.vae_cfg, self.text_kind, self.random_init = ZImageConfig(), VaeConfig(), "qwen3", None
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            raw = json.loads(cfg_path.read_text())
            if "dit" in raw:
                self.dit_cfg = ZImageConfig.from_json(raw["dit"])
            if "vae" in raw:
                v = dict(raw["vae"])
                if "ch_mult" in v:
                    v["ch_mult"] = tuple(v["ch_mult"])
                self.vae_cfg = VaeConfig(**v)
            self.text_kind = raw.get("text", self.text_kind)
            self.random_init = raw.get("random_init")
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = ZImageConfig.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32

    def load_text(self):
        if self.text_kind == "hash":
            return HashCaptionEncoder(self.dit_cfg.cap_feat_dim, self.device, self.dtype)
        from ..io.safetensors_io import load_dir
        from ..models.config import ModelConfig
        from ..models.text_encoders import CausalLmTextEncoder

        te, tk = self.root / "text_encoder", self.root / "tokenizer" / "tokenizer.json"
        if not te.is_dir() or not tk.exists():
            raise LoadError(f"{self.variant.value}: snapshot {self.root} lacks text_encoder/ or tokenizer/tokenizer.json")
        tok = TextTokenizer.from_file(tk, TokenizerConfig(max_length=MAX_PROMPT_TOKENS,
                                                          chat_template=PromptTemplate.QWEN_INSTRUCT))
        return QwenCaptionEncoder(CausalLmTextEncoder(ModelConfig.from_dir(te), load_dir(te), self.device), tok)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir

        if self.random_init is not None and self.backend == "b200":
            from ..models.dit_zimage import ZImageDiTGpu
            from ..models.vae import VaeDecoderGpu

            seed = int(self.random_init)
            return _Heavy(ZImageDiTGpu(self.dit_cfg, self.device).init_random(seed),
                          VaeDecoderGpu(self.vae_cfg, self.device).init_random(seed + 1))
        for d in ("transformer", "vae"):
            if not (self.root / d).is_dir():
                raise LoadError(f"{self.variant.value}: snapshot {self.root} lacks {d}/")
        dit_w = load_dir(self.root / "transformer")
        for ad in getattr(self, "adapters", []):          # low-rank adapters are merged into the weights at load
            from ..io.safetensors_io import load_file
            from .train import merge_lora

            if not Path(ad.path).is_file():
                raise LoadError(f"{self.variant.value}: adapter file {ad.path} not found")
            dit_w = merge_lora(dit_w, load_file(ad.path), ad.scale if ad.scale is not None else 1.0)
        vae_w = convert_diffusers_vae_decoder(load_dir(self.root / "vae"), len(self.vae_cfg.ch_mult))
        if self.backend == "b200":
            from ..models.dit_zimage import ZImageDiTGpu
            from ..models.vae import VaeDecoderGpu

            return _Heavy(ZImageDiTGpu(self.dit_cfg, self.device).load_state_dict(dit_w),
                          VaeDecoderGpu(self.vae_cfg, self.device).load_state_dict(vae_w))
        return _Heavy(OracleZImageDiT(self.dit_cfg, dit_w, device=self.device),
                      OracleVaeDecoder(self.vae_cfg, vae_w, device=self.device))

    def encode_reference(self, image: Image, width: int, height: int) -> torch.Tensor:
        from ..io.safetensors_io import load_dir

        return encode_reference_image(self.vae_cfg, convert_diffusers_vae_encoder(load_dir(self.root / "vae")), image, width,
                                      height, self.device, self.variant.value)

    def guidance(self, req: GenerationRequest) -> float | None:
        if self.variant is ZImageVariant.TURBO:
            return None
        g = req.true_cfg if req.true_cfg is not None else req.guidance
        return float(g) if g is not None else self.variant.default_guidance

    def encode(self, text, req: GenerationRequest):
        g = self.guidance(req)
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt or "") if g is not None and g > 1.0 else None
        return pos, neg

    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        v = self.variant
        steps = req.steps or v.default_steps
        guidance = self.guidance(req)
        base_seed = req.seed if req.seed is not None else default_seed()
        lh, lw = req.height // 8, req.width // 8
        dev, dt = self.device, self.dtype
        native = z_image_sigmas(v, steps)
        if req.scheduler is None:
            sigmas = native
        else:
            sigmas = schedule_sigmas(req.scheduler, FlowModelSampling(mu=req.scheduler_shift or 0.0), steps)
        ref = reference_of(req, v.value)
        clean, start = None, 0
        if ref is not None and init_time_step(steps, ref[1]) > 0:
            start = min(init_time_step(steps, ref[1]), len(sigmas) - 2)
            clean = self.encode_reference(ref[0], req.width, req.height).to(dev)
            sigmas = sigmas[start:]                    # the run enters the schedule at sigma_start
        solver, ops, ms = get_solver(req.sampler or "euler"), TorchLatentOps(), FlowModelSampling()
        gpu = self.backend == "b200"
        p = self.dit_cfg.patch_size
        # the caption branch of the DiT does not depend on the timestep: the device path runs it once per prompt
        caps = []
        for emb in cond:
            if emb is None:
                continue
            if gpu:
                tokens = heavy.dit.refine_caption(emb)
                caps.append((tokens, heavy.dit.rope_tables(lh // p, lw // p, tokens.shape[0])))
            else:
                caps.append((emb.to(dev, dt), None))

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
                tt = torch.full((1,), 1.0 - float(sigma), device=dev)
                outs = []
                for cap, ropes in caps:
                    o = heavy.dit.forward_graphed(x_in, tt, cap, ropes) if gpu else heavy.dit.forward(x_in, tt, cap)
                    outs.append(-o.float())
                vel = outs[0] if len(outs) == 1 else outs[1] + (outs[0] - outs[1]) * guidance
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
            if gpu:
                host = heavy.vae.decode_rgb8(z)[0].cpu()
            else:
                img = heavy.vae.decode(z)[0].permute(1, 2, 0)
                host = torch.round((img.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).cpu()
            return Image(width=req.width, height=req.height, pixels=host.contiguous().numpy().tobytes())

        return for_each_image_seed(base_seed, req.count, one_image)


def z_image_descriptor(variant: ZImageVariant, backend: str, prefix: str = "") -> ModelDescriptor:
    cfg = variant is ZImageVariant.BASE
    return ModelDescriptor(
        id=prefix + variant.value, family="z-image", backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=cfg, supports_guidance=cfg, supports_true_cfg=cfg,
            conditioning=[ConditioningKind.REFERENCE],
            supports_lora=True, supports_lokr=False, samplers=list(SOLVERS), schedulers=list(SCHEDULERS),
            supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8,
            supports_sequential_offload=True),
        required_components=[])


class ZImageGenerator(Generator):
    def __init__(self, pipe: ZImagePipeline, descriptor: ModelDescriptor, policy: OffloadPolicy):
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
            raise InferenceError(f"{mid}: steps must be >= 1 (an explicit 0 renders undenoised noise)")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} "
                                 f"(got {req.width}x{req.height})")

    def generate(self, req: GenerationRequest, on_progress: Callable = lambda p: None) -> GenerationOutput:
        self.validate(req)
        images = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(images=images)


def _load(variant: ZImageVariant, backend: str, prefix: str) -> Callable[[LoadSpec], ZImageGenerator]:
    def load(spec: LoadSpec) -> ZImageGenerator:
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
        pipe = ZImagePipeline(variant, Path(spec.weights.path), backend, device)
        pipe.adapters = list(spec.adapters)
        return ZImageGenerator(pipe, z_image_descriptor(variant, backend, prefix), spec.offload_policy)
    return load


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=(lambda v=v: z_image_descriptor(v, backend, prefix)), load=_load(v, backend, prefix))
            for v in (ZImageVariant.BASE, ZImageVariant.TURBO)]


def write_synthetic_snapshot(root, seed: int = 0, text: str = "hash", te_head_dim: int = 32) -> Path:
    """A tiny random Z-Image-shaped snapshot in the diffusers directory layout. text="hash" uses the weight-free
    caption encoder; text="qwen3" also writes a 3-layer random Qwen3 decoder and a toy byte-level BPE tokenizer with
    the chat template's role markers as special tokens."""
    from ..io.safetensors_io import save_file
    from ..models.dit_zimage import random_zimage_weights
    from ..models.vae import random_vae_weights

    root = Path(root)
    cap_dim = 64 if text == "hash" else 2 * te_head_dim
    dit = ZImageConfig(dim=384, n_layers=2, n_refiner_layers=1, n_heads=3, cap_feat_dim=cap_dim)
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_zimage_weights(dit, seed).items()},
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    from ..models.vae import random_vae_encoder_weights

    vae_sd = native_vae_to_diffusers(random_vae_weights(vae, seed + 1), len(vae.ch_mult))
    vae_sd.update(native_vae_encoder_to_diffusers(random_vae_encoder_weights(vae, seed + 3)))
    save_file({k: v.bfloat16() for k, v in vae_sd.items()}, root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": {"dim": dit.dim, "n_layers": dit.n_layers, "n_refiner_layers": dit.n_refiner_layers,
                "n_heads": dit.n_heads, "cap_feat_dim": dit.cap_feat_dim},
        "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks}, "text": text}))
    if text == "qwen3":
        _write_synthetic_qwen3(root, cap_dim, te_head_dim, seed + 2)
    return root


def native_vae_encoder_to_diffusers(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Inverse of convert_diffusers_vae_encoder (synthetic snapshots)."""
    out = {}
    attn = {"norm": "group_norm", "q": "to_q", "k": "to_k", "v": "to_v", "proj_out": "to_out.0"}
    for k, v in sd.items():
        r = k[len("encoder."):]
        if r.startswith("norm_out."):
            nk = "conv_norm_out." + r[len("norm_out."):]
        elif r.startswith("mid.block_"):
            i, rest = r[len("mid.block_"):].split(".", 1)
            nk = f"mid_block.resnets.{int(i) - 1}.{rest}"
        elif r.startswith("mid.attn_1."):
            name, leaf = r[len("mid.attn_1."):].rsplit(".", 1)
            nk = f"mid_block.attentions.0.{attn[name]}.{leaf}"
            if leaf == "weight" and name != "norm":
                v = v.reshape(v.shape[0], v.shape[1])
        elif r.startswith("down."):
            lvl, rest = r[len("down."):].split(".", 1)
            nk = f"down_blocks.{lvl}.resnets.{rest[len('block.'):]}" if rest.startswith("block.") else \
                f"down_blocks.{lvl}.downsamplers.0.conv.{rest[len('downsample.conv.'):]}"
        else:
            nk = r
        out["encoder." + nk.replace("nin_shortcut", "conv_shortcut")] = v
    return out


def _write_synthetic_qwen3(root: Path, hidden: int, head_dim: int, seed: int) -> None:
    import tokenizers
    from tokenizers import decoders, models, pre_tokenizers, trainers

    from ..io.safetensors_io import save_file
    from ..models.config import ModelConfig
    from ..models.oracle import random_llama_weights

    tok = tokenizers.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    corpus = ["a red fox jumps over the lazy dog", "user assistant", "a lighthouse at dusk, oil painting",
              "blurry low quality", "the quick brown fox"]
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|im_start|>", "<|im_end|>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    (root / "tokenizer").mkdir(exist_ok=True)
    tok.save(str(root / "tokenizer" / "tokenizer.json"))
    cfg_json = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": hidden,
                "intermediate_size": 2 * hidden, "num_hidden_layers": 3, "num_attention_heads": 2,
                "num_key_value_heads": 1, "head_dim": head_dim, "vocab_size": tok.get_vocab_size(),
                "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 1024,
                "tie_word_embeddings": True}
    (root / "text_encoder").mkdir(exist_ok=True)
    (root / "text_encoder" / "config.json").write_text(json.dumps(cfg_json))
    w = random_llama_weights(ModelConfig.from_json(cfg_json), seed, std=0.08)
    save_file({k: v.bfloat16() for k, v in w.items()}, root / "text_encoder" / "model.safetensors")
