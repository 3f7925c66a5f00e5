"""FLUX.1 text-to-image providers: `flux1_dev` / `flux1_schnell` on the sm_100a kernels and `cpu_flux1_*` on the
fp32 oracle (parity: candle-gen-flux/src/lib.rs:130-374, pipeline.rs:101-126,622-723,878-970).

generate(): validate -> residency.run(encode text -> for each image: seeded CPU noise -> patchify 2x2 -> flow
schedule with resolution-dependent shift (dev) -> sampler loop calling the DiT once per step (guidance is an
embedding input, no CFG batch) -> unpatchify -> VAE decode -> RGB8 on the host).

Snapshot layout: `<transformer_file>` (BFL key names) + `ae.safetensors`; an optional `swb_config.json`
({"dit": {...FluxConfig fields}, "vae": {...VaeConfig fields}, "text": "hash"}) overrides the fixed FLUX.1
dimensions - used by synthetic snapshots so conformance suites run in seconds."""
from __future__ import annotations

import enum
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, GenerationOutput, GenerationRequest, Generator, Modality,
                                            ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import PerComponentBytes, Registration
from ..contracts.gen_core.traits import reject_unknown_components
from ..contracts.gen_core.runtime import AdapterKind, LoadSpec, OffloadPolicy, ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import (SCHEDULERS, SOLVERS, FlowModelSampling, TorchLatentOps, build_flow_sigmas,
                                           compute_mu, denoise, get_solver, image_seq_len, schedule_sigmas)
from ..models.dit_flux import FluxConfig, OracleFluxDiT, make_ids, rope_table
from ..models.vae import OracleVaeDecoder, VaeConfig
from .residency import Residency
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw
from .text_encoders import HashTextEncoders, TextConditioning

SIZE_MULTIPLE = 16
FLUX1_DEV_ID, FLUX1_SCHNELL_ID = "flux1_dev", "flux1_schnell"


class Variant(enum.Enum):
    SCHNELL = "schnell"
    DEV = "dev"

    @property
    def model_id(self) -> str:
        return FLUX1_DEV_ID if self is Variant.DEV else FLUX1_SCHNELL_ID

    @property
    def default_steps(self) -> int:
        return 25 if self is Variant.DEV else 4

    @property
    def supports_guidance(self) -> bool:
        return self is Variant.DEV

    @property
    def default_guidance(self) -> float:
        return 3.5

    @property
    def t5_max_len(self) -> int:
        return 512 if self is Variant.DEV else 256

    @property
    def transformer_file(self) -> str:
        return "flux1-dev.safetensors" if self is Variant.DEV else "flux1-schnell.safetensors"


def flux_descriptor(variant: Variant, backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + variant.model_id, family="flux", backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=False, supports_guidance=variant.supports_guidance, supports_true_cfg=False,
            conditioning=[ConditioningKind.REFERENCE], supports_lora=True, supports_lokr=False, samplers=list(SOLVERS),
            schedulers=list(SCHEDULERS), supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8,
            supports_sequential_offload=True),
        required_components=[])


def patchify(z: torch.Tensor) -> torch.Tensor:
    """[1, 16, h, w] -> [1, (h/2)(w/2), 64], channel-major inside a patch (c, ph, pw)."""
    b, c, h, w = z.shape
    return z.view(b, c, h // 2, 2, w // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(b, (h // 2) * (w // 2), c * 4)


def unpatchify(x: torch.Tensor, h: int, w: int) -> torch.Tensor:
    b, _, d = x.shape
    c = d // 4
    return x.view(b, h // 2, w // 2, c, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(b, c, h, w)


def flux_schedule(variant: Variant, steps: int, width: int, height: int) -> list[float]:
    """steps+1 sigmas from 1 to 0; dev shifts time by mu(image sequence length) (pipeline.rs:101-126)."""
    if variant is Variant.DEV:
        return build_flow_sigmas(steps, compute_mu(image_seq_len(width, height), steps))
    return [1.0 - i / steps for i in range(steps + 1)]


@dataclass
class _Heavy:
    dit: Any
    vae: Any
    device: torch.device
    dtype: torch.dtype


class FluxPipeline:
    """Paths and configuration only; components are built by the residency owner when first needed."""

    def __init__(self, variant: Variant, root: Path, backend: str, device: torch.device):
        self.variant, self.root, self.backend, self.device = variant, Path(root), backend, device
        self.dit_cfg = FluxConfig(guidance_embed=variant.supports_guidance)
        self.vae_cfg = VaeConfig()
        self.text_kind = "t5_clip"
        self.random_init = None
        self.adapters: list = []
        self.pid_spec: tuple[Path, Path] | None = None       # (PiD checkpoint file, Gemma-2 snapshot directory)
        self._pid_engine = None
        # when set to a dict, render() records device-timed phases of the last image into it:
        # "step_ms" (one entry per model evaluation) and "vae_ms" (CUDA events; read after the image is on the host)
        self.timings: dict | None = None
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            raw = json.loads(cfg_path.read_text())
            if "dit" in raw:
                d = dict(raw["dit"])
                if "axes_dim" in d:
                    d["axes_dim"] = tuple(d["axes_dim"])
                self.dit_cfg = FluxConfig(**d)
            if "vae" in raw:
                v = dict(raw["vae"])
                if "ch_mult" in v:
                    v["ch_mult"] = tuple(v["ch_mult"])
                self.vae_cfg = VaeConfig(**v)
            self.text_kind = raw.get("text", self.text_kind)
            self.random_init = raw.get("random_init")      # seed: build random weights on the device, read no files
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32

    # ---- loaders -------------------------------------------------------------------------------------
    def load_text(self):
        if self.text_kind == "hash":
            return HashTextEncoders(self.dit_cfg.context_in_dim, self.dit_cfg.vec_in_dim, self.device, self.dtype)
        from .t5_clip import load_t5_clip

        return load_t5_clip(self.root, self.backend, self.device)

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_file

        if self.random_init is not None and self.backend == "b200":
            from ..models.dit_flux import FluxDiTGpu
            from ..models.vae import VaeDecoderGpu

            from ..parallel import default_communicator

            seed = int(self.random_init)
            comm = default_communicator()      # a multi-GPU job renders sequence parallel: every rank calls generate
            if comm is not None and (not comm.is_parallel or comm.device != self.device):
                comm = None
            return _Heavy(FluxDiTGpu(self.dit_cfg, comm=comm, device=self.device).init_random(seed),
                          VaeDecoderGpu(self.vae_cfg, self.device).init_random(seed + 1), self.device, self.dtype)
        tf = self.root / self.variant.transformer_file
        ae = self.root / "ae.safetensors"
        for p in (tf, ae):
            if not p.exists():
                raise LoadError(f"{self.variant.model_id}: missing weight file {p}")
        dit_w, vae_w = load_file(tf), load_file(ae)
        for ad in self.adapters:                         # low-rank adapters are merged into the weights at load
            from .train import merge_lora

            if not Path(ad.path).is_file():
                raise LoadError(f"{self.variant.model_id}: adapter file {ad.path} not found")
            dit_w = merge_lora(dit_w, load_file(ad.path), ad.scale if ad.scale is not None else 1.0)
        if self.backend == "b200":
            from ..models.dit_flux import FluxDiTGpu
            from ..models.vae import VaeDecoderGpu

            dit = FluxDiTGpu(self.dit_cfg, device=self.device).load_state_dict(dit_w)
            vae = VaeDecoderGpu(self.vae_cfg, self.device).load_state_dict(vae_w)
        else:
            dit = OracleFluxDiT(self.dit_cfg, dit_w, device=self.device)
            vae = OracleVaeDecoder(self.vae_cfg, vae_w, device=self.device)
        return _Heavy(dit, vae, self.device, self.dtype)

    def pid_engine(self, use_pid: bool):
        """The super-resolving pixel decoder of this latent space, loaded the first time a request asks for it (a spec
        the caller passed is never read by requests that do not use it)."""
        if not use_pid or self.pid_spec is None:
            return None
        if self._pid_engine is None:
            from .pid import PidEngine

            self._pid_engine = PidEngine.load(self.pid_spec[0], self.pid_spec[1], "flux", self.backend)
        return self._pid_engine

    # ---- phases --------------------------------------------------------------------------------------
    def encode(self, text, prompt: str) -> TextConditioning:
        return text.encode(prompt, self.variant.t5_max_len)

    def render(self, heavy: _Heavy, cond: TextConditioning, req: GenerationRequest, on_progress) -> list[Image]:
        v = self.variant
        steps = req.steps or v.default_steps
        guidance = (req.guidance if req.guidance is not None else v.default_guidance) if v.supports_guidance else None
        base_seed = req.seed if req.seed is not None else default_seed()
        lh, lw = req.height // 8, req.width // 8
        dev, dt = heavy.device, heavy.dtype
        txt = cond.txt.to(dev, dt)
        pooled = cond.pooled.to(dev, dt)
        txt_ids, img_ids = make_ids(lh // 2, lw // 2, txt.shape[1], dev)
        rope = rope_table(torch.cat([txt_ids, img_ids], 0), self.dit_cfg.axes_dim, self.dit_cfg.theta)
        ms = FlowModelSampling()
        if req.scheduler is None:
            sigmas = flux_schedule(v, steps, req.width, req.height)
        else:
            sigmas = schedule_sigmas(req.scheduler, FlowModelSampling(mu=req.scheduler_shift or 0.0), steps)
        from .reference import encode_reference_image, init_time_step, reference_of

        ref = reference_of(req, v.model_id)
        clean, start = None, 0
        if ref is not None and init_time_step(steps, ref[1]) > 0:
            from ..io.safetensors_io import load_file

            start = min(init_time_step(steps, ref[1]), len(sigmas) - 2)
            latents = encode_reference_image(self.vae_cfg, load_file(self.root / "ae.safetensors"), ref[0], req.width,
                                             req.height, dev, v.model_id)
            clean = patchify(latents).to(dev)
            sigmas = sigmas[start:]                    # the run enters the schedule at sigma_start
        solver = get_solver(req.sampler or "euler")
        ops = TorchLatentOps()
        gvec = torch.full((1,), float(guidance), device=dev) if guidance is not None else None
        c_lat = self.vae_cfg.z_channels

        events = [] if (self.timings is not None and self.backend == "b200") else None
        from .pid import check_pid_request, resolve_pid_decoder

        pid = self.pid_engine(req.use_pid)
        if req.use_pid:
            check_pid_request(pid, req, v.model_id)       # no engine / capture not wired / over budget: refused before any step
        pid_for = lambda seed: resolve_pid_decoder(pid, req, seed, v.model_id)                 # noqa: E731

        def one_image(seed: int) -> Image:
            if events is not None:
                events.clear()
            noise = seeded_noise_nchw(seed, c_lat, lh, lw)                    # CPU draw -> device
            x = patchify(noise).to(dev)
            if clean is not None:                       # x_t = (1 - sigma) clean + sigma noise at the entry point
                x = (1.0 - sigmas[0]) * clean + sigmas[0] * x.float()
            x = x.to(dt).contiguous()
            state = {"step": start}
            for s_done in range(1, start + 1):
                on_progress(ProgressStep(s_done, steps))

            def run_model(x_in, t):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{v.model_id}: cancelled at step {state['step']}")
                tt = torch.full((1,), float(t), device=dev)
                if self.backend == "b200":
                    if events is not None:
                        events.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
                        events[-1][0].record()
                    out = heavy.dit.forward_graphed(x_in, img_ids, txt, txt_ids, tt, pooled, gvec, rope=rope)
                    if events is not None:
                        events[-1][1].record()
                else:
                    out = heavy.dit.forward(x_in, img_ids, txt, txt_ids, tt, pooled, gvec)
                state["step"] += 1
                if state["step"] <= steps:          # multi-evaluation solvers still report `steps` events
                    on_progress(ProgressStep(state["step"], steps))
                return out.to(dt).contiguous()

            x = solver.sample(ops, ms, lambda xx, s: denoise(ops, ms, xx, s, run_model), x, sigmas, seed)
            while state["step"] < steps:            # solvers that skip the final evaluation at sigma 0
                state["step"] += 1
                on_progress(ProgressStep(state["step"], steps))
            if req.cancel.is_cancelled():
                raise Canceled(f"{v.model_id}: cancelled before decode")
            on_progress(ProgressDecoding())
            z = unpatchify(x.float(), lh, lw)
            if pid is not None:                      # the same latent the VAE would get; the image comes out `scale` x larger
                px = pid_for(seed).decode(z.cpu())[0].permute(1, 2, 0)
                host = torch.round((px.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).contiguous()
                return Image(width=host.shape[1], height=host.shape[0], pixels=host.numpy().tobytes())
            if self.backend == "b200":
                if events is not None:
                    v0, v1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    v0.record()
                u8 = heavy.vae.decode_rgb8(z)[0]                               # [H, W, 3] uint8 on device
                if events is not None:
                    v1.record()
                host = u8.cpu()
                if events is not None:
                    self.timings["step_ms"] = [a.elapsed_time(b) for a, b in events]
                    self.timings["vae_ms"] = v0.elapsed_time(v1)
            else:
                img = heavy.vae.decode(z)[0].permute(1, 2, 0)
                host = torch.round((img.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).cpu()
            return Image(width=req.width, height=req.height, pixels=host.contiguous().numpy().tobytes())

        return for_each_image_seed(base_seed, req.count, one_image)


class FluxGenerator(Generator):
    def __init__(self, variant: Variant, pipe: FluxPipeline, descriptor: ModelDescriptor, policy: OffloadPolicy):
        self.variant, self.pipe, self._descriptor = variant, pipe, descriptor
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
        images = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req.prompt),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(images=images)


def _load(variant: Variant, backend: str, prefix: str) -> Callable[[LoadSpec], FluxGenerator]:
    def load(spec: LoadSpec) -> FluxGenerator:
        mid = prefix + variant.model_id
        if spec.weights is None or spec.weights.is_file:
            raise Unsupported(f"{mid}: needs a snapshot directory (single-file checkpoints are not supported)")
        if spec.quantize is not None:
            raise Unsupported(f"{mid}: quantised loading ({spec.quantize.name}) is not supported")
        reject_unknown_components(spec.components, ["pid_gemma"], mid)
        pid_spec = None
        if spec.pid is not None or "pid_gemma" in spec.components:
            if spec.pid is None or not spec.pid.is_file or "pid_gemma" not in spec.components or spec.components["pid_gemma"].is_file:
                raise LoadError(f"{mid}: the pixel decoder needs LoadSpec.pid (the converted checkpoint file) and the "
                                "'pid_gemma' component (a Gemma-2 snapshot directory)")
            pid_spec = (Path(spec.pid.path), Path(spec.components["pid_gemma"].path))
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid}: control branches / IP adapters are not supported by this provider")
        for ad in spec.adapters:
            if ad.kind is not AdapterKind.LORA:
                raise Unsupported(f"{mid}: adapter kind {ad.kind.value} is not supported (lora)")
        if backend == "b200":
            if not torch.cuda.is_available():
                raise LoadError(f"{mid}: no CUDA device")
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
        pipe = FluxPipeline(variant, Path(spec.weights.path), backend, device)    # lazy: paths only
        pipe.adapters = list(spec.adapters)
        pipe.pid_spec = pid_spec
        return FluxGenerator(variant, pipe, flux_descriptor(variant, backend, prefix), spec.offload_policy)
    return load


def _footprint(variant: Variant) -> Callable[[LoadSpec], PerComponentBytes | None]:
    def footprint(spec: LoadSpec) -> PerComponentBytes | None:
        if spec.weights is None or spec.weights.is_file:
            return None
        root = Path(spec.weights.path)
        out = {}
        for name, rel in (("transformer", variant.transformer_file), ("vae", "ae.safetensors")):
            f = root / rel
            if f.exists():
                out[name] = f.stat().st_size
        te = PerComponentBytes.from_root_subdirs(root, {"text_encoder": "text_encoder", "text_encoder_2":
                                                        "text_encoder_2"})
        out.update(te.components)
        return PerComponentBytes(out)
    return footprint


def registrations(backend: str = "b200") -> list[Registration]:
    """`flux1_schnell` + `flux1_dev` for the sm_100a backend, `cpu_flux1_*` for the fp32 oracle backend."""
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=(lambda v=v: flux_descriptor(v, backend, prefix)), load=_load(v, backend, prefix),
                         footprint=_footprint(v)) for v in (Variant.SCHNELL, Variant.DEV)]


def write_synthetic_snapshot(root, variant: Variant = Variant.DEV, seed: int = 0, text: str = "hash") -> Path:
    """A tiny random FLUX-shaped snapshot (2+2 blocks, hidden 256). text="hash" uses the weight-free prompt encoder;
    text="t5_clip" also writes tiny random T5 / CLIP encoders with real tokenizer files (a SentencePiece model trained
    on a toy corpus, a toy CLIP BPE vocabulary) in the Hugging Face directory layout."""
    from ..io.safetensors_io import save_file
    from ..models.dit_flux import random_flux_weights
    from ..models.vae import random_vae_weights

    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    dit = FluxConfig(in_channels=64, vec_in_dim=32, context_in_dim=64, hidden_size=256, num_heads=2, depth=2,
                     depth_single=2, guidance_embed=variant.supports_guidance)
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1)
    save_file({k: v.bfloat16() for k, v in random_flux_weights(dit, seed).items()}, root / variant.transformer_file)
    from ..models.vae import random_vae_encoder_weights

    save_file({k: v.bfloat16() for k, v in {**random_vae_weights(vae, seed + 1), **random_vae_encoder_weights(vae, seed + 3)}.items()},
              root / "ae.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": {**{k: getattr(dit, k) for k in ("in_channels", "vec_in_dim", "context_in_dim", "hidden_size",
                                                "num_heads", "depth", "depth_single", "guidance_embed")},
                "axes_dim": list(dit.axes_dim)},
        "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks}, "text": text}))
    if text == "t5_clip":
        _write_synthetic_text_encoders(root, dit.context_in_dim, dit.vec_in_dim, seed)
    return root


def _write_synthetic_text_encoders(root: Path, context_dim: int, vec_dim: int, seed: int) -> None:
    import sentencepiece as spm

    from ..io.safetensors_io import save_file

    g = torch.Generator().manual_seed(seed + 7)
    rnd = lambda *shape: torch.randn(*shape, generator=g) * 0.05   # noqa: E731
    # ---- T5 (2 layers, d_model = context_dim) --------------------------------------------------------------
    (root / "tokenizer_2").mkdir(exist_ok=True)
    corpus = root / "tokenizer_2" / "corpus.txt"
    words = "a fox cat dog red blue green big small runs jumps over the lazy quick brown photo of in on".split()
    corpus.write_text("\n".join(" ".join(words[(i * 7 + j) % len(words)] for j in range(6)) for i in range(200)))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(root / "tokenizer_2" / "spiece"), vocab_size=64,
                                   model_type="unigram", pad_id=0, eos_id=1, unk_id=2, bos_id=-1,
                                   minloglevel=2, hard_vocab_limit=False)
    corpus.unlink()
    t5 = {"vocab_size": 64, "d_model": context_dim, "d_kv": 16, "d_ff": 96, "num_layers": 2, "num_heads": 4,
          "relative_attention_num_buckets": 8, "relative_attention_max_distance": 32}
    tw = {"shared.weight": rnd(64, context_dim), "encoder.final_layer_norm.weight": torch.ones(context_dim),
          "encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight": rnd(8, 4)}
    for i in range(2):
        p = f"encoder.block.{i}.layer"
        for n in "qkv":
            tw[f"{p}.0.SelfAttention.{n}.weight"] = rnd(64, context_dim)
        tw[f"{p}.0.SelfAttention.o.weight"] = rnd(context_dim, 64)
        tw[f"{p}.0.layer_norm.weight"] = torch.ones(context_dim)
        tw[f"{p}.1.layer_norm.weight"] = torch.ones(context_dim)
        tw[f"{p}.1.DenseReluDense.wi_0.weight"] = rnd(96, context_dim)
        tw[f"{p}.1.DenseReluDense.wi_1.weight"] = rnd(96, context_dim)
        tw[f"{p}.1.DenseReluDense.wo.weight"] = rnd(context_dim, 96)
    (root / "text_encoder_2").mkdir(exist_ok=True)
    (root / "text_encoder_2" / "config.json").write_text(json.dumps(t5))
    save_file(tw, root / "text_encoder_2" / "model.safetensors")
    # ---- CLIP (2 layers, hidden = vec_dim) ------------------------------------------------------------------
    from .text_models import _bytes_to_unicode

    chars = sorted(set(_bytes_to_unicode().values()))
    vocab = {}
    for c in chars:
        vocab[c] = len(vocab)
    for c in chars:
        vocab[c + "</w>"] = len(vocab)
    merges = [("f", "o"), ("fo", "x</w>"), ("c", "a"), ("ca", "t</w>"), ("d", "o"), ("do", "g</w>")]
    for a, b in merges:
        vocab[a + b] = len(vocab)
    vocab["<|startoftext|>"] = len(vocab)
    vocab["<|endoftext|>"] = len(vocab)
    (root / "tokenizer").mkdir(exist_ok=True)
    (root / "tokenizer" / "vocab.json").write_text(json.dumps(vocab), encoding="utf-8")
    (root / "tokenizer" / "merges.txt").write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges),
                                                   encoding="utf-8")
    V, Hc = len(vocab), vec_dim
    clip = {"vocab_size": V, "hidden_size": Hc, "intermediate_size": 2 * Hc, "num_hidden_layers": 2,
            "num_attention_heads": 2, "max_position_embeddings": 24, "eos_token_id": vocab["<|endoftext|>"],
            "hidden_act": "quick_gelu"}
    cw = {"text_model.embeddings.token_embedding.weight": rnd(V, Hc),
          "text_model.embeddings.position_embedding.weight": rnd(24, Hc),
          "text_model.final_layer_norm.weight": torch.ones(Hc), "text_model.final_layer_norm.bias": torch.zeros(Hc)}
    for i in range(2):
        lp = f"text_model.encoder.layers.{i}."
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            cw[f"{lp}self_attn.{n}.weight"], cw[f"{lp}self_attn.{n}.bias"] = rnd(Hc, Hc), rnd(Hc)
        for n in ("layer_norm1", "layer_norm2"):
            cw[f"{lp}{n}.weight"], cw[f"{lp}{n}.bias"] = torch.ones(Hc), torch.zeros(Hc)
        cw[lp + "mlp.fc1.weight"], cw[lp + "mlp.fc1.bias"] = rnd(2 * Hc, Hc), rnd(2 * Hc)
        cw[lp + "mlp.fc2.weight"], cw[lp + "mlp.fc2.bias"] = rnd(Hc, 2 * Hc), rnd(Hc)
    (root / "text_encoder").mkdir(exist_ok=True)
    (root / "text_encoder" / "config.json").write_text(json.dumps(clip))
    save_file(cw, root / "text_encoder" / "model.safetensors")
