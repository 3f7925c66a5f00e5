"""SenseNova-U1 text-to-image providers `sensenova_u1_8b` (50 steps, guidance 4) and `sensenova_u1_8b_fast` (8 steps, no
guidance; the 8-step distillation LoRA is merged into the generation path at load) (parity:
candle-gen-sensenova/src/{lib,t2i,text,distill}.rs).

The prompt is rendered as a chat query (a fixed system message, the user turn, an empty think block and the image-start
tag) and prefilled once on the understanding path; the unconditional branch prefills the bare query with no system
message. Sampling runs in pixel space from seeded noise scaled with the resolution (sqrt(tokens / 64), capped at 8), over
`steps` Euler steps on a sigma-shifted time grid from 0 to 1 (shift 3 unless the checkpoint declares its own or the
request overrides it); the guided velocity is uncond + scale * (cond - uncond). Sizes are multiples of 32.
The distillation LoRA comes from the `distill_lora` component, or the file of the same name inside the snapshot; a
snapshot carrying `distill_merged.json` already has it folded in."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import Capabilities, GenerationOutput, GenerationRequest, Generator, Modality, ModelDescriptor
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec, ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import SOLVERS  # noqa: F401  (the model has its own Euler loop: no sampler menu)
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.sensenova import (NeoChatConfig, SenseNovaT2i, image_indexes, merge_distill_lora, random_sensenova_weights, time_schedule,
                                unpatchify)
from .family import rgb8_image
from .seed import default_seed, for_each_image_seed, seeded_normal

MODEL_ID, MODEL_ID_FAST, FAMILY = "sensenova_u1_8b", "sensenova_u1_8b_fast", "sensenova"
DEFAULT_STEPS, DEFAULT_GUIDANCE, DEFAULT_STEPS_FAST, DEFAULT_GUIDANCE_FAST = 50, 4.0, 8, 1.0
DEFAULT_TIMESTEP_SHIFT, SIZE_MULTIPLE, T_EPS = 3.0, 32, 0.02
DISTILL_LORA_FILE, DISTILL_MERGED_MARKER, DISTILL_COMPONENT = "SenseNova-U1-8B-MoT-LoRA-8step-V1.0.safetensors", "distill_merged.json", "distill_lora"
SYSTEM_MESSAGE_FOR_GEN = (
    "You are an image generation and editing assistant that accurately understands and executes user intent.\n\nYou support two "
    "modes:\n\n1. Think Mode:\nIf the task requires reasoning, you MUST start with a <think></think> block. Put all reasoning inside "
    "the block using plain text. DO NOT include any image tags. Keep it reasonable and directly useful for producing the final "
    "image.\n\n2. Non-Think Mode:\nIf no reasoning is needed, directly produce the final image.\n\nTask Types:\n\nA. Text-to-Image "
    "Generation:\n- Generate a high-quality image based on the user's description.\n- Ensure visual clarity, semantic consistency, "
    "and completeness.\n- DO NOT introduce elements that contradict or override the user's intent.\n\nB. Image Editing:\n- Use the "
    "provided image(s) as input or reference for modification or transformation.\n- The result can be an edited image or a new "
    "image based on the reference(s).\n- Preserve all unspecified attributes unless explicitly changed.\n\nGeneral Rules:\n- For any "
    "visible text in the image, follow the language specified for the rendered text in the user's description, not the language "
    "of the prompt. If no language is specified, use the user's input language.")


def build_neo1_query(prompt: str, system_message: str) -> str:
    head = f"<|im_start|>system\n{system_message}<|im_end|>\n" if system_message else ""
    return f"{head}<|im_start|>user\n{prompt}<|im_end|>\n<|im_start|>assistant\n"


def cond_query(prompt: str) -> str:
    return build_neo1_query(prompt, SYSTEM_MESSAGE_FOR_GEN) + "<think>\n\n</think>\n\n<img>"


def uncond_query() -> str:
    return build_neo1_query("", "") + "<img>"


def sensenova_descriptor(backend: str, prefix: str = "", fast: bool = False) -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + (MODEL_ID_FAST if fast else MODEL_ID), family=FAMILY, backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=False, supports_guidance=True, supports_true_cfg=False, conditioning=[], supports_lora=False,
            supports_lokr=False, samplers=[], schedulers=[], supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8,
            supports_kv_cache=True),
        required_components=[])


class SenseNovaGenerator(Generator):
    def __init__(self, root: Path, backend: str, prefix: str, fast: bool, distill_lora: Path | None):
        self.root, self.backend, self.fast, self.distill_lora = Path(root), backend, fast, distill_lora
        self._descriptor = sensenova_descriptor(backend, prefix, fast)
        self._model = None

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        self._descriptor.capabilities.validate_request(mid, req)
        if not req.prompt.strip():
            raise InferenceError(f"{mid}: prompt must not be empty")
        if req.steps == 0:
            raise InferenceError(f"{mid}: steps must be >= 1")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")

    def model(self):
        if self._model is None:
            import tokenizers

            from ..io.safetensors_io import load_file

            cj, tk = self.root / "config.json", self.root / "tokenizer.json"
            if not cj.is_file():
                raise LoadError(f"{self._descriptor.id}: {cj} missing")
            if not tk.is_file():
                raise LoadError(f"missing {tk}: the snapshot ships only vocab.json + merges.txt; materialise the fast tokenizer.json first")
            try:
                cfg = NeoChatConfig.from_json(json.loads(cj.read_text(encoding="utf-8")))
            except ValueError as e:
                raise LoadError(str(e)) from e
            weights: dict[str, torch.Tensor] = {}
            for f in sorted(self.root.glob("*.safetensors")):
                if f.name != DISTILL_LORA_FILE:
                    weights.update(load_file(f))
            if "language_model.model.embed_tokens.weight" not in weights:
                raise LoadError(f"{self._descriptor.id}: no model weights (*.safetensors) under {self.root}")
            if self.distill_lora is not None:
                n = merge_distill_lora(weights, load_file(self.distill_lora), cfg.llm.num_hidden_layers)
                expected = 7 * cfg.llm.num_hidden_layers + 2
                if n != expected:
                    raise LoadError(f"{self._descriptor.id}: distill LoRA merged {n} targets, expected {expected} (wrong LoRA file?)")
            dev = "cuda" if self.backend == "b200" else "cpu"
            dt = torch.bfloat16 if self.backend == "b200" else torch.float32
            self._model = (SenseNovaT2i(cfg, weights, dt, dev), tokenizers.Tokenizer.from_file(str(tk)), cfg)
        return self._model

    def options(self, req: GenerationRequest, cfg: NeoChatConfig) -> dict:
        steps, guidance = (DEFAULT_STEPS_FAST, DEFAULT_GUIDANCE_FAST) if self.fast else (DEFAULT_STEPS, DEFAULT_GUIDANCE)
        return dict(cfg_scale=req.guidance if req.guidance is not None else guidance, num_steps=req.steps or steps,
                    timestep_shift=float(req.scheduler_shift) if req.scheduler_shift is not None
                    else cfg.inference_timestep_shift(DEFAULT_TIMESTEP_SHIFT))

    @torch.no_grad()
    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        self.validate(req)
        model, tok, cfg = self.model()
        o = self.options(req, cfg)
        ids = lambda text: tok.encode(text, add_special_tokens=True).ids            # noqa: E731
        cache_c, len_c = model.prefill(ids(cond_query(req.prompt)))
        guided = o["cfg_scale"] > 1.0
        cache_u, len_u = model.prefill(ids(uncond_query())) if guided else (None, 0)
        cell, ps = model.cell, cfg.patch_size
        th, tw = req.height // cell, req.width // cell
        L, steps = th * tw, o["num_steps"]
        times = time_schedule(steps, o["timestep_shift"])
        scale = model.noise_scale_for(req.height // ps, req.width // ps)
        noise_embed = model.noise_scale_embed(scale, L)
        prep_c = model.prepare(*image_indexes(th, tw, len_c), cache_c.len)
        prep_u = model.prepare(*image_indexes(th, tw, len_u), cache_u.len) if guided else None

        def one(seed: int):
            img = seeded_normal(seed, 3 * req.height * req.width).view(1, 3, req.height, req.width) * scale
            for i in range(steps):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{self._descriptor.id}: cancelled at step {i}")
                t, t_next = times[i], times[i + 1]
                z, cond = model.step_tokens(img, t, noise_embed)
                v = model.predict_v(cond, prep_c, cache_c, z, t, T_EPS)
                if guided:
                    vu = model.predict_v(cond, prep_u, cache_u, z, t, T_EPS)
                    v = vu + (v - vu) * o["cfg_scale"]
                img = unpatchify((z.to(v.device) + v * (t_next - t)).cpu().float(), cell, th, tw)
                on_progress(ProgressStep(i + 1, steps))
            on_progress(ProgressDecoding())
            return [rgb8_image(img[0], req.width, req.height)]

        base = req.seed if req.seed is not None else default_seed()
        return GenerationOutput(images=[im for ims in for_each_image_seed(base, req.count, one) for im in ims])


def resolve_distill_lora(spec: LoadSpec, root: Path, mid: str) -> Path:
    src = spec.components.get(DISTILL_COMPONENT)
    if src is not None:
        if not src.is_file:
            raise LoadError(f"{mid}: the '{DISTILL_COMPONENT}' component must be the {DISTILL_LORA_FILE} .safetensors file, not a directory: {src.path}")
        if not Path(src.path).exists():
            raise LoadError(f"{mid}: the '{DISTILL_COMPONENT}' component path does not exist: {src.path}")
        return Path(src.path)
    if (root / DISTILL_LORA_FILE).exists():
        return root / DISTILL_LORA_FILE
    raise LoadError(f"{mid}: distill LoRA `{DISTILL_LORA_FILE}` not found - stage the '{DISTILL_COMPONENT}' component in "
                    f"LoadSpec.components or co-locate the file in the snapshot dir {root}")


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"

    def loader(fast: bool):
        def load(spec: LoadSpec) -> SenseNovaGenerator:
            mid = prefix + (MODEL_ID_FAST if fast else MODEL_ID)
            if spec.weights is None or spec.weights.is_file:
                raise LoadError(f"{mid}: expects a snapshot directory (config.json + *.safetensors + tokenizer.json)")
            if spec.quantize is not None:
                raise Unsupported(f"{mid}: on-the-fly quantization is not supported")
            if spec.adapters:
                raise Unsupported(f"{mid}: user-supplied adapters are not supported (supports_lora=false)")
            if spec.control or spec.extra_controls or spec.ip_adapter:
                raise Unsupported(f"{mid}: control / IP-adapter overlays are not supported")
            reject_unknown_components(spec.components, [DISTILL_COMPONENT] if fast else [], mid)
            root = Path(spec.weights.path)
            lora = None
            if fast and not (root / DISTILL_MERGED_MARKER).exists():
                lora = resolve_distill_lora(spec, root, mid)
            if backend == "b200" and not torch.cuda.is_available():
                raise LoadError(f"{mid}: no CUDA device")
            return SenseNovaGenerator(root, backend, prefix, fast, lora)
        return load

    return [Registration(descriptor=(lambda f=f: sensenova_descriptor(backend, prefix, f)), load=loader(f)) for f in (False, True)]


def write_synthetic_snapshot(root, seed: int = 0, lora: bool = True) -> Path:
    """Tiny random snapshot (2 layers of width 32, 4-pixel patches merged 2 x 2) with a toy byte-level tokenizer that knows
    the chat markup, and a rank-2 distillation LoRA under the published file name."""
    import tokenizers
    from tokenizers import decoders, models, pre_tokenizers, trainers

    from ..io.safetensors_io import save_file
    from ..models.sensenova import NeoLlmConfig, NeoVisionConfig

    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    tok = tokenizers.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(["a red fox jumps over the lazy dog", SYSTEM_MESSAGE_FOR_GEN],
                            trainers.BpeTrainer(vocab_size=330, special_tokens=["<|im_start|>", "<|im_end|>", "<think>", "</think>", "<img>"],
                                                initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tok.save(str(root / "tokenizer.json"))
    llm = dict(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=16,
               vocab_size=tok.get_vocab_size())
    vis = dict(hidden_size=16, llm_hidden_size=32, patch_size=16)
    (root / "config.json").write_text(json.dumps({"model_type": "neo_chat", "patch_size": 16, "downsample_ratio": 0.5, "timestep_shift": 1.0,
                                                  "llm_config": llm, "vision_config": vis}))
    cfg = NeoChatConfig(patch_size=16, llm=NeoLlmConfig(**llm), vision=NeoVisionConfig(**vis))
    save_file(random_sensenova_weights(cfg, seed), root / "model.safetensors")
    if lora:
        g = torch.Generator().manual_seed(seed + 9)
        full = random_sensenova_weights(cfg, seed)
        lw: dict[str, torch.Tensor] = {}
        targets = ["fm_modules.fm_head.0", "fm_modules.fm_head.2"]
        for i in range(2):
            p = f"language_model.model.layers.{i}"
            targets += [f"{p}.self_attn.{n}_proj_mot_gen" for n in "qkvo"] + [f"{p}.mlp_mot_gen.{n}_proj" for n in ("gate", "up", "down")]
        for t in targets:
            o, i_ = full[t + ".weight"].shape
            lw[t + ".lora_down.weight"], lw[t + ".lora_up.weight"] = torch.randn(2, i_, generator=g) * 0.1, torch.randn(o, 2, generator=g) * 0.1
            lw[t + ".alpha"] = torch.tensor(2.0)
        save_file(lw, root / DISTILL_LORA_FILE)
    return root
