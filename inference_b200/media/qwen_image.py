"""Qwen-Image text-to-image provider `qwen_image` (and `cpu_qwen_image` on the fp32 oracle)
(parity: candle-gen-qwen-image/src/lib.rs, pipeline.rs, text_encoder.rs, config.rs).

generate(): the prompt is wrapped in the image-description chat template and run through the Qwen2.5-VL language
model; the last layer's normed hidden states, minus the template's first 34 tokens, are the text features. Sampling is
flow-match Euler over `steps` sigmas from 1 to 1/steps, shifted by exp(mu) with mu linear in the image token count and
stretched so the last non-zero sigma is 0.02. Guidance is true CFG with a norm rescale: comb = neg + g (pos - neg),
scaled per token to the norm of pos (default g = 4, negative prompt " "). Latents are 16-channel, packed 2x2 like FLUX;
the autoencoder is the single-frame reading of the Qwen-Image video autoencoder.

Snapshot layout (diffusers): `transformer/`, `text_encoder/` + `tokenizer/tokenizer.json`, `vae/`; `swb_config.json`
overrides dimensions for synthetic snapshots."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, GenerationOutput, GenerationRequest, Generator, Modality,
                                            ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import AdapterKind, LoadSpec, OffloadPolicy, ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import (SCHEDULERS, SOLVERS, FlowModelSampling, TorchLatentOps, denoise, get_solver,
                                           schedule_sigmas)
from ..contracts.gen_core.tokenizer import PromptTemplate, TextTokenizer, TokenizerConfig
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.dit_flux import rope_table
from ..models.dit_qwen_image import OracleQwenImageDiT, QwenImageConfig, position_ids
from ..models.vae_qwen import QwenVaeConfig, QwenVaeDecoder
from .flux import SIZE_MULTIPLE, patchify, unpatchify
from .residency import Residency
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw

MODEL_ID = "qwen_image"
DEFAULT_STEPS, DEFAULT_GUIDANCE, NEGATIVE_FALLBACK = 30, 4.0, " "
PROMPT_DROP_TOKENS, MAX_PROMPT_TOKENS = 34, 1024 + 34
BASE_SHIFT, MAX_SHIFT, BASE_SEQ, MAX_SEQ, SHIFT_TERMINAL = 0.5, 0.9, 256.0, 8192.0, 0.02


def qwen_mu(width: int, height: int) -> float:
    seq = (width // 16) * (height // 16)
    m = (MAX_SHIFT - BASE_SHIFT) / (MAX_SEQ - BASE_SEQ)
    return seq * m + (BASE_SHIFT - m * BASE_SEQ)


def qwen_sigmas(steps: int, width: int, height: int) -> list[float]:
    n = max(1, steps)
    ramp = [1.0 if n == 1 else 1.0 + (1.0 / n - 1.0) * i / (n - 1) for i in range(n)]
    e = math.exp(qwen_mu(width, height))
    shifted = [e / (e + (1.0 / s - 1.0)) for s in ramp]
    scale = (1.0 - shifted[-1]) / (1.0 - SHIFT_TERMINAL)
    return [1.0 - (1.0 - s) / scale for s in shifted] + [0.0]


def guided_velocity(pos: torch.Tensor, neg: torch.Tensor, guidance: float) -> torch.Tensor:
    """neg + g (pos - neg), rescaled per token so its norm over channels equals that of pos."""
    comb = neg + (pos - neg) * guidance
    return comb * (pos.norm(dim=-1, keepdim=True) / comb.norm(dim=-1, keepdim=True).clamp_min(1e-12))


def language_model_weights(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The language-model tensors of a Qwen2.5-VL checkpoint under plain decoder names (the vision tower is dropped)."""
    out = {}
    for k, v in sd.items():
        if k.startswith(("visual.", "model.visual.")):
            continue
        out[k.replace("model.language_model.", "model.").replace("language_model.model.", "model.")] = v
    return out


def language_model_config(j: dict):
    from ..models.config import ModelConfig

    t = {**{k: v for k, v in j.items() if k not in ("vision_config", "text_config")}, **j.get("text_config", {})}
    t.update({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2"})
    t.pop("rope_scaling", None)                         # text-only prompts: the three M-RoPE sections coincide
    return ModelConfig.from_json(t)


class QwenVlCaptionEncoder:
    def __init__(self, encoder, tokenizer: TextTokenizer, drop: int = PROMPT_DROP_TOKENS):
        self.encoder, self.tok, self.drop = encoder, tokenizer, drop

    def encode(self, prompt: str) -> torch.Tensor:
        ids = self.tok.encode_chat_ids(prompt, True)[:MAX_PROMPT_TOKENS]
        if len(ids) <= self.drop:
            raise InferenceError(f"{MODEL_ID}: the templated prompt has {len(ids)} tokens, not more than the "
                                 f"{self.drop} template tokens that are dropped")
        return self.encoder.encode(ids)[:, self.drop:]


class HashCaptionEncoder:
    def __init__(self, dim: int, device, dtype):
        from .text_encoders import HashTextEncoders

        self.h = HashTextEncoders(dim, 8, device, dtype)

    def encode(self, prompt: str) -> torch.Tensor:
        return self.h.encode(prompt, 8 + len(prompt.encode("utf-8"))).txt


@dataclass
class _Heavy:
    dit: Any
    vae: Any


class QwenImagePipeline:
    def __init__(self, root: Path, backend: str, device: torch.device):
        self.root, self.backend, self.device = Path(root), backend, device
        self.dit_cfg, self.vae_cfg, self.text_kind, self.random_init = QwenImageConfig(), QwenVaeConfig(), "qwen_vl", None
        self.drop, self.adapters = PROMPT_DROP_TOKENS, []
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            raw = json.loads(cfg_path.read_text())
            if "dit" in raw:
                self.dit_cfg = QwenImageConfig.from_json(raw["dit"])
            if "vae" in raw:
                v = dict(raw["vae"])
                if "dim_mult" in v:
                    v["dim_mult"] = tuple(v["dim_mult"])
                self.vae_cfg = QwenVaeConfig(**v)
            self.text_kind = raw.get("text", self.text_kind)
            self.random_init = raw.get("random_init")
            self.drop = int(raw.get("prompt_drop_tokens", self.drop))
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = QwenImageConfig.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32

    def load_text(self):
        if self.text_kind == "hash":
            return HashCaptionEncoder(self.dit_cfg.joint_attention_dim, self.device, self.dtype)
        from ..io.safetensors_io import load_dir
        from ..models.text_encoders import CausalLmTextEncoder

        te, tk = self.root / "text_encoder", self.root / "tokenizer" / "tokenizer.json"
        if not (te / "config.json").is_file() or not tk.exists():
            raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks text_encoder/config.json or tokenizer/tokenizer.json")
        cfg = language_model_config(json.loads((te / "config.json").read_text()))
        enc = CausalLmTextEncoder(cfg, language_model_weights(load_dir(te)), self.device, skip_last=0, final_norm=True)
        tok = TextTokenizer.from_file(tk, TokenizerConfig(max_length=MAX_PROMPT_TOKENS, chat_template=PromptTemplate.QWEN_IMAGE))
        return QwenVlCaptionEncoder(enc, tok, self.drop)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir, load_file
        from ..models.vae_qwen import random_qwen_vae_weights

        gpu = self.backend == "b200"
        if self.random_init is not None and gpu:
            from ..models.dit_qwen_image import QwenImageDiTGpu

            seed = int(self.random_init)
            return _Heavy(QwenImageDiTGpu(self.dit_cfg, device=self.device).init_random(seed),
                          QwenVaeDecoder(self.vae_cfg, random_qwen_vae_weights(self.vae_cfg, seed + 1), self.dtype, self.device))
        for d in ("transformer", "vae"):
            if not (self.root / d).is_dir():
                raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks {d}/")
        dit_w = load_dir(self.root / "transformer")
        for ad in self.adapters:
            from .train import merge_lora

            if not Path(ad.path).is_file():
                raise LoadError(f"{MODEL_ID}: adapter file {ad.path} not found")
            dit_w = merge_lora(dit_w, load_file(ad.path), ad.scale if ad.scale is not None else 1.0)
        vae = QwenVaeDecoder(self.vae_cfg, load_dir(self.root / "vae"), self.dtype, self.device)
        if gpu:
            from ..models.dit_qwen_image import QwenImageDiTGpu

            return _Heavy(QwenImageDiTGpu(self.dit_cfg, device=self.device).load_state_dict(dit_w), vae)
        return _Heavy(OracleQwenImageDiT(self.dit_cfg, dit_w, device=self.device), vae)

    @staticmethod
    def guidance(req: GenerationRequest) -> float:
        g = req.true_cfg if req.true_cfg is not None else req.guidance
        return float(g) if g is not None else DEFAULT_GUIDANCE

    def encode(self, text, req: GenerationRequest):
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt or NEGATIVE_FALLBACK) if self.guidance(req) > 1.0 else None
        return pos, neg

    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        steps = req.steps or DEFAULT_STEPS
        guidance = self.guidance(req)
        base_seed = req.seed if req.seed is not None else default_seed()
        lh, lw = req.height // 8, req.width // 8
        dev, dt = self.device, self.dtype
        fc = self.dit_cfg.flux_config()
        if req.scheduler is None:
            sigmas = qwen_sigmas(steps, req.width, req.height)
        else:
            sigmas = schedule_sigmas(req.scheduler, FlowModelSampling(mu=req.scheduler_shift or qwen_mu(req.width, req.height)),
                                     steps)
        solver, ops, ms = get_solver(req.sampler or "euler"), TorchLatentOps(), FlowModelSampling()
        gpu = self.backend == "b200"
        branches = []
        for emb in cond:
            if emb is None:
                continue
            txt = heavy.dit.prepare_text(emb.to(dev, dt))           # the pre-norm does not depend on the step
            txt_ids, img_ids = position_ids(lh // 2, lw // 2, txt.shape[1], dev)
            branches.append((txt, txt_ids, img_ids, rope_table(torch.cat([txt_ids, img_ids], 0), fc.axes_dim, fc.theta)))

        def one_image(seed: int) -> Image:
            x = patchify(seeded_noise_nchw(seed, self.vae_cfg.z_dim, lh, lw)).to(dev, dt).contiguous()
            state = {"step": 0}

            def run_model(x_in, sigma):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{MODEL_ID}: cancelled at step {state['step']}")
                tt = torch.full((1,), float(sigma), device=dev)
                outs = []
                for txt, txt_ids, img_ids, rope in branches:
                    if gpu:
                        o = heavy.dit.forward_graphed(x_in, img_ids, txt, txt_ids, tt, None, None, rope=rope)
                    else:
                        o = heavy.dit.forward(x_in, img_ids, txt, txt_ids, tt, None, None)
                    outs.append(o.float())
                vel = outs[0] if len(outs) == 1 else guided_velocity(outs[0], outs[1], guidance)
                state["step"] += 1
                if state["step"] <= steps:
                    on_progress(ProgressStep(state["step"], steps))
                return vel.to(dt).contiguous()

            x = solver.sample(ops, ms, lambda xx, s: denoise(ops, ms, xx, s, run_model), x, sigmas, seed)
            while state["step"] < steps:
                state["step"] += 1
                on_progress(ProgressStep(state["step"], steps))
            if req.cancel.is_cancelled():
                raise Canceled(f"{MODEL_ID}: cancelled before decode")
            on_progress(ProgressDecoding())
            img = heavy.vae.decode(unpatchify(x.float(), lh, lw))[0].float().permute(1, 2, 0)
            host = torch.round((img.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).cpu()
            return Image(width=req.width, height=req.height, pixels=host.contiguous().numpy().tobytes())

        return for_each_image_seed(base_seed, req.count, one_image)


def qwen_image_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family="qwen-image", backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=True, conditioning=[],
            supports_lora=True, supports_lokr=False, samplers=list(SOLVERS), schedulers=list(SCHEDULERS),
            supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8,
            supports_sequential_offload=True),
        required_components=[])


class QwenImageGenerator(Generator):
    def __init__(self, pipe: QwenImagePipeline, descriptor: ModelDescriptor, policy: OffloadPolicy):
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
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} "
                                 f"(got {req.width}x{req.height})")

    def generate(self, req: GenerationRequest, on_progress: Callable = lambda p: None) -> GenerationOutput:
        self.validate(req)
        images = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(images=images)


def _load(backend: str, prefix: str) -> Callable[[LoadSpec], QwenImageGenerator]:
    def load(spec: LoadSpec) -> QwenImageGenerator:
        mid = prefix + MODEL_ID
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
        pipe = QwenImagePipeline(Path(spec.weights.path), backend, device)
        pipe.adapters = list(spec.adapters)
        return QwenImageGenerator(pipe, qwen_image_descriptor(backend, prefix), spec.offload_policy)
    return load


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=lambda: qwen_image_descriptor(backend, prefix), load=_load(backend, prefix))]


def write_synthetic_snapshot(root, seed: int = 0, text: str = "hash", te_head_dim: int = 32) -> Path:
    """A tiny random Qwen-Image-shaped snapshot in the diffusers directory layout. text="qwen_vl" also writes a 2-layer
    random Qwen2 decoder under Qwen2.5-VL key names (with a stub vision tensor that loading must ignore) and a toy
    tokenizer; the number of dropped template tokens is then 2 instead of 34."""
    from ..io.safetensors_io import save_file
    from ..models.dit_qwen_image import random_qwen_image_weights
    from ..models.vae_qwen import random_qwen_vae_weights

    root = Path(root)
    cap_dim = 64 if text == "hash" else 2 * te_head_dim
    dit = QwenImageConfig(num_layers=2, num_attention_heads=2, joint_attention_dim=cap_dim)
    vae = QwenVaeConfig(base_dim=16, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_qwen_image_weights(dit, seed).items()},
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    save_file({k: v.bfloat16() for k, v in random_qwen_vae_weights(vae, seed + 1).items()},
              root / "vae" / "diffusion_pytorch_model.safetensors")
    cfg = {"dit": {"num_layers": dit.num_layers, "num_attention_heads": dit.num_attention_heads,
                   "joint_attention_dim": dit.joint_attention_dim},
           "vae": {"base_dim": vae.base_dim, "dim_mult": list(vae.dim_mult), "num_res_blocks": vae.num_res_blocks},
           "text": text}
    if text == "qwen_vl":
        cfg["prompt_drop_tokens"] = 2
        _write_synthetic_qwen_vl(root, cap_dim, te_head_dim, seed + 2)
    (root / "swb_config.json").write_text(json.dumps(cfg))
    return root


def _write_synthetic_qwen_vl(root: Path, hidden: int, head_dim: int, seed: int) -> None:
    import tokenizers
    from tokenizers import decoders, models, pre_tokenizers, trainers

    from ..io.safetensors_io import save_file
    from ..models.oracle import random_llama_weights

    tok = tokenizers.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    corpus = ["a red fox jumps over the lazy dog", "system user assistant", "a lighthouse at dusk, oil painting",
              "Describe the image by detailing the color, shape, size, texture, quantity, text, spatial relationships"]
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|im_start|>", "<|im_end|>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    (root / "tokenizer").mkdir(exist_ok=True)
    tok.save(str(root / "tokenizer" / "tokenizer.json"))
    text_cfg = {"hidden_size": hidden, "intermediate_size": 2 * hidden, "num_hidden_layers": 2, "num_attention_heads": 2,
                "num_key_value_heads": 1, "head_dim": head_dim, "vocab_size": tok.get_vocab_size(), "rms_norm_eps": 1e-6,
                "rope_theta": 1000000.0, "max_position_embeddings": 2048, "tie_word_embeddings": False,
                "rope_scaling": {"type": "mrope", "mrope_section": [4, 6, 6]}}
    top = {"architectures": ["Qwen2_5_VLForConditionalGeneration"], "model_type": "qwen2_5_vl", "text_config": text_cfg,
           "vision_config": {"depth": 1}}
    (root / "text_encoder").mkdir(exist_ok=True)
    (root / "text_encoder" / "config.json").write_text(json.dumps(top))
    w = random_llama_weights(language_model_config(top), seed, std=0.08)
    out = {k.replace("model.", "model.language_model.", 1) if k.startswith("model.") else k: v.bfloat16() for k, v in w.items()}
    out["model.visual.patch_embed.proj.weight"] = torch.zeros(4, 4, dtype=torch.bfloat16)
    save_file(out, root / "text_encoder" / "model.safetensors")
