"""Vision providers: CLIP image / text embedders and the LLaVA-style captioner
(candle-gen-clip `clip_vit_l14`, `clip_vit_l14_text`; candle-gen-joycaption: SigLIP tower + projector + Llama).

Embedders return L2-normalised joint-space vectors (image and text land in one space, so their dot product is the
similarity). The captioner encodes the image with the vision tower, projects the patch states into the language
model's embedding space, substitutes them for the `<image>` placeholder tokens of the chat prompt and decodes
greedily - on the B200 backend through the paged-KV engine (embedding override on the prefill step), on the CPU
backend through the fp32 oracle."""
from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.nn.functional as F

from ..contracts.errors import LoadError
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec
from ..contracts.gen_core.traits import Captioner, ImageEmbedder, SimpleDescriptor, TextEmbedder
from ..models.text_encoders import ClipTextConfig, ClipTextEncoder, linear
from ..models.vision import CLIP_MEAN, CLIP_STD, SIGLIP_MEAN, SIGLIP_STD, VisionConfig, VisionTower, preprocess


def image_tensor(img: Image) -> torch.Tensor:
    return torch.frombuffer(bytearray(img.pixels), dtype=torch.uint8).view(img.height, img.width, 3)


def _device_dtype(backend: str):
    return ("cuda", torch.bfloat16) if backend == "b200" else ("cpu", torch.float32)


def _load_dir(spec: LoadSpec, what: str) -> tuple[Path, dict, dict[str, torch.Tensor]]:
    from ..io.safetensors_io import load_dir

    if spec.weights is None or spec.weights.is_file:
        raise LoadError(f"{what}: the load spec needs a snapshot directory")
    d = Path(spec.weights.path)
    if not (d / "config.json").is_file():
        raise LoadError(f"{what}: {d}/config.json not found")
    return d, json.loads((d / "config.json").read_text()), load_dir(d)


class ClipImageEmbedder(ImageEmbedder):
    ID = "clip_vit_l14"

    def __init__(self, tower: VisionTower, backend: str):
        self.tower, self.backend = tower, backend

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "clip", self.backend, {"dim": self.tower.cfg.projection_dim})

    def embed(self, images: list[Image]) -> list[list[float]]:
        if not images:
            return []
        px = torch.cat([preprocess(image_tensor(i), self.tower.cfg.image_size, CLIP_MEAN, CLIP_STD) for i in images])
        e = self.tower.image_embeds(px).float()
        return F.normalize(e, dim=-1).cpu().tolist()


class ClipTextEmbedder(TextEmbedder):
    ID = "clip_vit_l14_text"

    def __init__(self, enc: ClipTextEncoder, proj: torch.Tensor | None, tokenizer, backend: str):
        self.enc, self.proj, self.tok, self.backend = enc, proj, tokenizer, backend

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "clip", self.backend, {})

    def embed(self, texts: list[str]) -> list[list[float]]:
        if not texts:
            return []
        ids = torch.tensor([self.tok.encode(t) for t in texts], dtype=torch.int64)
        _, pooled = self.enc.encode(ids)
        e = linear(pooled, self.proj) if self.proj is not None else pooled
        return F.normalize(e.float(), dim=-1).cpu().tolist()


class LlavaCaptioner(Captioner):
    """vision tower -> `multi_modal_projector` (linear, GELU, linear) -> language model."""

    ID = "llava_captioner"
    DEFAULT_PROMPT = "Write a descriptive caption for this image."

    def __init__(self, tower: VisionTower, proj: dict[str, torch.Tensor], lm, tokenizer, image_token_id: int,
                 backend: str, feature_layer: int = -2, drop_cls: bool | None = None, stop_ids: tuple[int, ...] = ()):
        self.tower, self.proj, self.lm, self.tok = tower, proj, lm, tokenizer
        self.image_token_id, self.backend, self.feature_layer = image_token_id, backend, feature_layer
        self.drop_cls = tower.cfg.kind == "clip" if drop_cls is None else drop_cls
        self.stop_ids = stop_ids

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "llava", self.backend, {"vision": self.tower.cfg.kind})

    def image_features(self, image: Image) -> torch.Tensor:
        """[patches, lm_hidden]: the tower's states at `feature_layer` through the projector."""
        cfg = self.tower.cfg
        mean, std = (CLIP_MEAN, CLIP_STD) if cfg.kind == "clip" else (SIGLIP_MEAN, SIGLIP_STD)
        px = preprocess(image_tensor(image), cfg.image_size, mean, std, crop=cfg.kind == "clip")
        h = self.tower.hidden_states(px, self.feature_layer)[0]
        if self.drop_cls:
            h = h[1:]
        h = linear(h, self.proj["linear_1.weight"], self.proj.get("linear_1.bias"))
        h = F.gelu(h.float()).to(h.dtype)
        return linear(h, self.proj["linear_2.weight"], self.proj.get("linear_2.bias"))

    def build_prompt(self, prompt: str, n_image_tokens: int) -> list[int]:
        """Token ids with the single `<image>` placeholder expanded to one token per image feature."""
        ids = self.tok.encode(prompt)
        if self.image_token_id not in ids:
            ids = [self.image_token_id] + ids
        out: list[int] = []
        for t in ids:
            out += [self.image_token_id] * n_image_tokens if t == self.image_token_id else [t]
        return out

    def caption_tokens(self, image: Image, prompt: str | None = None, max_new_tokens: int = 256) -> list[int]:
        feats = self.image_features(image)
        ids = self.build_prompt(prompt or self.DEFAULT_PROMPT, feats.shape[0])
        pos = [i for i, t in enumerate(ids) if t == self.image_token_id]
        if len(pos) != feats.shape[0]:
            raise ValueError("the prompt must contain exactly one <image> placeholder")
        return self.lm.generate_with_embeds(ids, pos, feats, max_new_tokens, self.stop_ids)

    def caption(self, image: Image, prompt: str | None = None, max_new_tokens: int = 256) -> str:
        return self.tok.decode(self.caption_tokens(image, prompt, max_new_tokens)).strip()


class OracleLm:
    """Greedy decoding on the fp32 oracle with image features spliced into the prompt embeddings."""

    def __init__(self, oracle):
        self.oracle = oracle

    def generate_with_embeds(self, ids, positions, feats, max_new_tokens, stop_ids=()) -> list[int]:
        o = self.oracle
        emb = o.embed(torch.tensor([ids], dtype=torch.long, device=o.device)).clone()
        emb[0, positions] = feats.to(emb.device, emb.dtype)
        cache = o.make_cache()
        logits = o.project_logits(o.hidden_states(None, cache, 0, embeds=emb)[:, -1:, :])[:, 0]
        out: list[int] = []
        for _ in range(max_new_tokens):
            tok = int(torch.argmax(logits[0].float()))
            if tok in stop_ids:
                break
            out.append(tok)
            logits = o.decode_logits(torch.tensor([[tok]], dtype=torch.long), cache, cache.offset)
        return out


class EngineLm:
    """Greedy decoding on the paged-KV GPU engine: the prefill step overrides the placeholder rows' embeddings."""

    def __init__(self, engine):
        self.engine = engine

    def generate_with_embeds(self, ids, positions, feats, max_new_tokens, stop_ids=()) -> list[int]:
        runner = self.engine.runner
        seq = self.engine.new_sequence()
        try:
            tok = int(runner.prefill([seq], [ids], embed_overrides=[(positions, feats)])[0])
            out: list[int] = []
            for _ in range(max_new_tokens):
                if tok in stop_ids:
                    break
                out.append(tok)
                tok = int(runner.decode([seq], [tok])[0])
            return out
        finally:
            seq.release()


def _load_captioner(spec: LoadSpec, backend: str) -> LlavaCaptioner:
    """A Hugging Face LLaVA snapshot: config.json with vision_config / text_config / image_token_index, weights under
    `vision_tower.`, `multi_modal_projector.`, `language_model.` (with or without a leading `model.`)."""
    from ..contracts.core_llm.tokenizer import Tokenizer
    from ..models.config import ModelConfig

    d, cfg, w = _load_dir(spec, "llava captioner")
    dev, dtype = _device_dtype(backend)
    w = {(k[6:] if k.startswith("model.") and not k.startswith("model.layers") else k): v for k, v in w.items()}
    vis = {k[len("vision_tower."):]: v for k, v in w.items() if k.startswith("vision_tower.")}
    proj = {k[len("multi_modal_projector."):]: v.to(dev, dtype) for k, v in w.items()
            if k.startswith("multi_modal_projector.")}
    lmw = {}
    for k, v in w.items():
        if k.startswith("language_model."):
            k2 = k[len("language_model."):]
            lmw[k2 if k2.startswith(("model.", "lm_head.")) else "model." + k2] = v
    if "lm_head.weight" in w:
        lmw["lm_head.weight"] = w["lm_head.weight"]
    if not vis or not proj or not lmw:
        raise LoadError("llava captioner: the snapshot lacks vision_tower / multi_modal_projector / language_model weights")
    vcfg = VisionConfig.from_json(cfg)
    tower = VisionTower(vcfg, vis, dev, dtype)
    mcfg = ModelConfig.from_json(cfg["text_config"])
    if backend == "b200":
        from ..engine.llm_engine import EngineConfig, LlmEngine
        from ..models.llama import LlamaGpu

        model = LlamaGpu(mcfg, device=torch.device("cuda")).load_state_dict(lmw)
        lm = EngineLm(LlmEngine(model, EngineConfig(max_batch=1, max_seq_len=4096)))
    else:
        from ..models.oracle import OracleLlama

        lm = OracleLm(OracleLlama(mcfg, lmw, dtype=torch.float32, device="cpu"))
    tok = Tokenizer.from_file(d / "tokenizer.json")
    stop = tuple(i for i in (cfg.get("eos_token_id"), cfg["text_config"].get("eos_token_id")) if isinstance(i, int))
    return LlavaCaptioner(tower, proj, lm, tok, int(cfg.get("image_token_index", cfg.get("image_token_id", 0))), backend,
                          int(cfg.get("vision_feature_layer", -2)),
                          cfg.get("vision_feature_select_strategy", "default") == "default" and vcfg.kind == "clip",
                          stop)


def _load_clip_image(spec: LoadSpec, backend: str) -> ClipImageEmbedder:
    _, cfg, w = _load_dir(spec, ClipImageEmbedder.ID)
    dev, dtype = _device_dtype(backend)
    return ClipImageEmbedder(VisionTower(VisionConfig.from_json(cfg), w, dev, dtype), backend)


def _load_clip_text(spec: LoadSpec, backend: str) -> ClipTextEmbedder:
    from .text_models import ClipBpeTokenizer

    d, cfg, w = _load_dir(spec, ClipTextEmbedder.ID)
    dev, dtype = _device_dtype(backend)
    tcfg = ClipTextConfig.from_json(cfg.get("text_config", cfg))
    proj = w.get("text_projection.weight")
    return ClipTextEmbedder(ClipTextEncoder(tcfg, w, dev, dtype), proj.to(dev, dtype) if proj is not None else None,
                            ClipBpeTokenizer.from_dir(d, tcfg.max_position_embeddings), backend)


def registrations(backend: str) -> dict[str, list[Registration]]:
    d = lambda i, fam: (lambda: SimpleDescriptor(i, fam, backend, {}))
    return {
        "image_embedder": [Registration(d(ClipImageEmbedder.ID, "clip"), lambda s: _load_clip_image(s, backend))],
        "text_embedder": [Registration(d(ClipTextEmbedder.ID, "clip"), lambda s: _load_clip_text(s, backend))],
        "captioner": [Registration(d(LlavaCaptioner.ID, "llava"), lambda s: _load_captioner(s, backend))],
        "transform": [Registration(d(DepthTransform.ID, "depth_anything"), lambda s: _load_depth(s, backend))],
    }


class DepthTransform:
    """`Transform` provider: image -> depth map rendered as an 8-bit grey image of the input size (min-max
    normalised; larger = closer for relative-depth checkpoints)."""

    ID = "depth_anything_v2"

    def __init__(self, model, backend: str):
        self.model, self.backend = model, backend

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "depth_anything", self.backend, {"type": self.model.cfg.depth_estimation_type})

    def depth(self, image: Image, target: int | None = None) -> torch.Tensor:
        """fp32 [H, W] at the input resolution."""
        from ..models.depth import preprocess as depth_pre

        cfg = self.model.cfg
        px = depth_pre(image_tensor(image), target or cfg.image_size, cfg.patch_size)
        d = self.model.predict(px).float().unsqueeze(1)
        return F.interpolate(d, size=(image.height, image.width), mode="bilinear", align_corners=False)[0, 0].cpu()

    def apply(self, image: Image, params: dict | None = None) -> Image:
        d = self.depth(image, (params or {}).get("target"))
        lo, hi = float(d.min()), float(d.max())
        g = ((d - lo) / (hi - lo) if hi > lo else torch.zeros_like(d)).mul(255).round().clamp(0, 255).to(torch.uint8)
        return Image(image.width, image.height, bytes(g.unsqueeze(-1).expand(-1, -1, 3).contiguous().flatten().tolist()))


def _load_depth(spec: LoadSpec, backend: str) -> DepthTransform:
    from ..models.depth import DepthAnything, DepthConfig

    _, cfg, w = _load_dir(spec, DepthTransform.ID)
    dev, dtype = _device_dtype(backend)
    return DepthTransform(DepthAnything(DepthConfig.from_json(cfg), w, dev, dtype), backend)
