"""Text-LLM providers over the decode backends: `b200-llama` (sm_100a kernels, paged KV, tensor parallel) and
`cpu-llama` (fp32 oracle). Capability target: candle-llm/src/provider.rs:39-1285 (`candle-llama`): load an HF
snapshot directory or a GGUF file, render the chat template, tokenize, optional JSON constraint mask, thinking /
tool-call segmentation, stop strings, incremental detokenisation, typed cancel, usage accounting."""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Callable

import numpy as np
import torch

from ..contracts.core_llm import (Canceled, Channel, ChatMlTemplate, ChatTemplate, Constraint, DoneEvent,
                                  FinishReason, IncrementalDetok, JinjaChatTemplate, JsonConstraint, Llama3Template,
                                  LoadError, LoadSpec, Quantize, RenderOptions, StopMatcher, StreamEvent,
                                  TextLlm, TextLlmCapabilities, TextLlmDescriptor, TextLlmOutput,
                                  TextLlmRegistration, TextLlmRequest, ThinkingSegmenter, TokenEvent, Tokenizer,
                                  ToolCallSegmenter, Unsupported, Usage)
from ..io import gguf as gguf_io
from ..io import gguf_quants as gq
from ..io.safetensors_io import load_dir
from ..models.config import Architecture, ModelConfig
from ..models.oracle import OracleLlama
from ..policy.sampler import SamplingParams
from .backend import DecodeBackend, GpuBackend, OracleBackend
from .decode import GenerationConfig, generate

BACKEND_GPU = "b200"
BACKEND_CPU = "cpu"
_STOP_NAMES = ("<|eot_id|>", "<|end_of_text|>", "<|im_end|>", "<|endoftext|>", "</s>", "<end_of_turn>", "<|user|>")
_PROJ_SUFFIXES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "gate_proj.weight",
                  "up_proj.weight", "down_proj.weight", "qkv_proj.weight", "gate_up_proj.weight")


def quantize_roundtrip(w: torch.Tensor, bits: int) -> torch.Tensor:
    """Projection weight -> GGML Q4_K (bits 4) or Q8_0 (bits 8) blocks -> dense again: the numerics of a model
    quantised on load (candle-llm/src/primitives/projection.rs:15-53 maps Q4 -> Q4K, Q8 -> Q8_0)."""
    k = w.shape[-1]
    block = 256 if bits == 4 else 32
    if k % block:
        return w
    x = w.detach().float().cpu().numpy()
    raw = gq.quantize_q4_k(x) if bits == 4 else gq.quantize_q8_0(x)
    y = gq.dequantize(raw, "Q4_K" if bits == 4 else "Q8_0", x.size).reshape(x.shape)
    return torch.from_numpy(y.copy()).to(w.dtype)


def _read_json(p: Path) -> dict:
    try:
        return json.loads(p.read_text())
    except (OSError, json.JSONDecodeError):
        return {}


def _supported_on_gpu(cfg: ModelConfig) -> bool:
    return (cfg.head_dim == 128 and cfg.mla is None and
            cfg.architecture not in (Architecture.QWEN35, Architecture.DEEPSEEK_V2))


def probe_config(spec: LoadSpec) -> ModelConfig | None:
    """Weightless probe: config.json of a snapshot directory or the metadata of a GGUF file."""
    p = Path(spec.source)
    try:
        if p.is_dir() and (p / "config.json").is_file():
            return ModelConfig.from_dir(p)
        if p.is_file() and (p.suffix == ".gguf" or p.read_bytes()[:4] == b"GGUF"):
            ck = gguf_io.GgufCheckpoint(p)
            cfg = ModelConfig.from_json(ck.config())
            ck.file.close()
            return cfg
    except Exception:
        return None
    return None


class LlamaProvider(TextLlm):
    def __init__(self, descriptor: TextLlmDescriptor, backend: DecodeBackend, tokenizer: Tokenizer,
                 template: ChatTemplate, stop_tokens: list[int], cfg: ModelConfig):
        self._descriptor = descriptor
        self.backend = backend
        self.tokenizer = tokenizer
        self.template = template
        self.stop_tokens = stop_tokens
        self.cfg = cfg
        self._constraint_table = None

    # ---- loading ------------------------------------------------------------------------------------
    @staticmethod
    def load(spec: LoadSpec, provider_id: str, backend_name: str, comm=None) -> "LlamaProvider":
        p = Path(spec.source)
        if p.is_dir():
            cfg = ModelConfig.from_dir(p)
            weights = load_dir(p)
            tok_path = p / "tokenizer.json"
            if not tok_path.is_file():
                raise LoadError(f"{p}: tokenizer.json not found")
            tokenizer = Tokenizer.from_file(tok_path)
            tcfg = _read_json(p / "tokenizer_config.json")
            template, thinking, tools = _pick_template(tcfg.get("chat_template") and tcfg, cfg)
            extra_eos = _eos_ids(_read_json(p / "config.json")) | _eos_ids(_read_json(p / "generation_config.json"))
        elif p.is_file():
            ck = gguf_io.GgufCheckpoint(p)
            cfg = ModelConfig.from_json(ck.config())
            weights = ck.tensors()
            tj = ck.tokenizer_json()
            if tj is None:
                raise Unsupported(f"{p}: GGUF tokenizer model {ck.file.metadata.get('tokenizer.ggml.model')!r} "
                                  "cannot be reconstructed (byte-level BPE only)")
            tokenizer = Tokenizer.from_json(tj)
            ct = ck.chat_template()
            template, thinking, tools = _pick_template({"chat_template": ct} if ct else None, cfg)
            extra_eos = _eos_ids(ck.config())
        else:
            raise LoadError(f"model source '{spec.source}' is neither a snapshot directory nor a GGUF file")
        bits = spec.quantize.value if spec.quantize is not None else cfg.quantization_bits
        if bits in (4, 8):
            weights = {k: (quantize_roundtrip(v, bits) if k.endswith(_PROJ_SUFFIXES) else v) for k, v in weights.items()}
        stop = sorted(extra_eos | {i for n in _STOP_NAMES if (i := tokenizer.token_to_id(n)) is not None})
        backend = _build_backend(cfg, weights, backend_name, comm)
        caps = TextLlmCapabilities(max_context_tokens=backend.max_context, max_new_tokens=0, supports_system_prompt=True,
                                   supports_vision=False, supports_video=False, supports_thinking=thinking,
                                   supports_tools=tools, supported_constraints=[Constraint.JSON])
        d = TextLlmDescriptor(provider_id, cfg.architecture.family, backend_name, caps)
        return LlamaProvider(d, backend, tokenizer, template, stop, cfg)

    # ---- multimodal hooks (text-only here; the LLaVA provider overrides them) -----------------------------
    def _render_messages(self, req: TextLlmRequest):
        return req.messages

    def _splice_media(self, req: TextLlmRequest, prompt_ids: list[int]):
        """(token ids, sequence holding pending embedding overrides or None)."""
        return prompt_ids, None

    # ---- contract ---------------------------------------------------------------------------------------
    def descriptor(self) -> TextLlmDescriptor:
        return self._descriptor

    def validate(self, req: TextLlmRequest) -> None:
        self._descriptor.capabilities.validate_request(self._descriptor.id, req)

    def generate(self, req: TextLlmRequest, on_event: Callable[[StreamEvent], None]) -> TextLlmOutput:
        self.validate(req)
        if req.cancel.is_cancelled():
            raise Canceled()
        prompt = self.template.render_with(self._render_messages(req), RenderOptions(True, req.enable_thinking_kwarg(),
                                                                                     req.tools))
        prompt_ids = self.tokenizer.encode(prompt, add_special_tokens=False)
        prompt_ids, media_seq = self._splice_media(req, prompt_ids)
        if len(prompt_ids) + 1 > self.backend.max_context:
            from ..contracts.core_llm import InvalidRequest
            raise InvalidRequest(f"[{self._descriptor.id}] prompt of {len(prompt_ids)} tokens exceeds the context "
                                 f"window {self.backend.max_context}")
        s = req.sampling
        cfg = GenerationConfig(max_new_tokens=req.max_new_tokens,
                               sampling=SamplingParams(s.temperature, s.top_p, s.top_k, s.repetition_penalty,
                                                       s.repetition_context),
                               seed=req.seed if req.seed is not None else 0, stop_tokens=tuple(self.stop_tokens),
                               cancel=req.cancel)
        mask = self._json_mask() if req.constraint is Constraint.JSON else None
        caps = self._descriptor.capabilities
        seg = ThinkingSegmenter() if caps.supports_thinking else None
        if seg is not None and prompt.rstrip().endswith("<think>"):
            seg.push("<think>")
        tool_seg = ToolCallSegmenter(req.tools) if caps.supports_tools and req.tools else None
        stopper = StopMatcher(req.stop)
        st = _StreamState(on_event)
        acc: list[int] = []
        detok = IncrementalDetok()

        string_stop = [False]

        def route_content(text: str, tid: int) -> bool:
            pieces = tool_seg.push(text) if tool_seg is not None else [text]
            for piece in pieces:
                chunk = stopper.push(piece)
                if chunk.emit:
                    st.emit(tid, chunk.emit, Channel.CONTENT)
                if chunk.stop:
                    string_stop[0] = True
                    return False
            return True

        def sink(tok: int) -> bool:
            acc.append(tok)
            delta = detok.push(self.tokenizer.decode(acc, skip_special_tokens=True))
            if delta is None:
                return True
            if seg is None:
                return route_content(delta, tok)
            for span in seg.push(delta):
                if span.channel is Channel.THINKING:
                    st.emit(tok, span.text, Channel.THINKING)
                elif not route_content(span.text, tok):
                    return False
            return True

        try:
            res = generate(self.backend, prompt_ids, cfg, sink, mask, seq=media_seq)
        finally:
            if media_seq is not None:
                self.backend.release(media_seq)
        if not string_stop[0]:
            # end-of-generation tails, in pipeline order: reasoning segmenter, tool segmenter, stop matcher
            if seg is not None:
                for span in seg.flush():
                    if span.channel is Channel.THINKING:
                        st.emit(st.last_id, span.text, Channel.THINKING)
                    else:
                        route_content(span.text, st.last_id)
            if tool_seg is not None and not string_stop[0]:
                for piece in tool_seg.flush():
                    c = stopper.push(piece)
                    if c.emit:
                        st.emit(st.last_id, c.emit, Channel.CONTENT)
            tail = stopper.flush()
            if tail and not string_stop[0]:
                st.emit(st.last_id, tail, Channel.CONTENT)
        usage = Usage(len(prompt_ids), len(res.tokens))
        on_event(DoneEvent(res.finish_reason, usage))
        return TextLlmOutput(text=st.content, thinking=st.thinking or None,
                             tool_calls=tool_seg.take_calls() if tool_seg is not None else [], usage=usage,
                             finish_reason=res.finish_reason)

    def _json_mask(self):
        if self._constraint_table is None:
            self._constraint_table = self.tokenizer.constraint_decode_table()
        jc = JsonConstraint(self._constraint_table)
        consumed = [0]
        stops = self.stop_tokens

        def mask(generated: list[int]):
            while consumed[0] < len(generated):
                jc.accept(generated[consumed[0]])
                consumed[0] += 1
            allowed = np.asarray(jc.allowed(), dtype=np.uint8)
            if jc.can_stop():
                for s in stops:
                    if s < allowed.size:
                        allowed[s] = 1
            if not allowed.any():           # nothing extends the value: only stopping remains
                for s in stops:
                    if s < allowed.size:
                        allowed[s] = 1
            return allowed

        return mask


class _StreamState:
    def __init__(self, on_event):
        self.on_event = on_event
        self.index = 0
        self.last_id = 0
        self.content = ""
        self.thinking = ""

    def emit(self, tid: int, text: str, channel: Channel) -> None:
        if channel is Channel.CONTENT:
            self.content += text
        else:
            self.thinking += text
        self.last_id = tid
        self.on_event(TokenEvent(tid, text, self.index, channel))
        self.index += 1


def _eos_ids(cfg: dict) -> set[int]:
    e = cfg.get("eos_token_id")
    if isinstance(e, int):
        return {e}
    if isinstance(e, list):
        return {int(x) for x in e if isinstance(x, int)}
    return set()


def _pick_template(tokenizer_config: dict | None, cfg: ModelConfig) -> tuple[ChatTemplate, bool, bool]:
    """Jinja template from the tokenizer config when present, else a built-in layout by family. The template
    source decides whether thinking (`enable_thinking`) and tools (`tool_call`) are advertised."""
    if tokenizer_config:
        try:
            t = JinjaChatTemplate.from_tokenizer_config(tokenizer_config)
            return t, "enable_thinking" in t.source, "tool_call" in t.source
        except Exception:
            pass
    if cfg.architecture in (Architecture.QWEN3, Architecture.QWEN3_VL, Architecture.QWEN2_MOE):
        return ChatMlTemplate(), False, False
    return Llama3Template(), False, False


def _build_backend(cfg: ModelConfig, weights: dict, backend_name: str, comm=None) -> DecodeBackend:
    if cfg.architecture is Architecture.QWEN35:
        # hybrid Gated-DeltaNet decoder: its own model class (recurrent state instead of a paged KV cache); on the
        # b200 backend it runs in bf16 on the device with its projections on the tcgen05 GEMM
        from ..models.qwen35 import Qwen35Config, Qwen35Model

        on_gpu = backend_name == BACKEND_GPU
        if on_gpu and not torch.cuda.is_available():
            raise LoadError("the b200 backend needs a CUDA device (use the cpu runtime bundle on hosts without one)")
        qcfg = Qwen35Config.from_json(cfg.raw)
        model = Qwen35Model(qcfg, weights, dtype=torch.bfloat16 if on_gpu else torch.float32,
                            device="cuda" if on_gpu else "cpu")
        return OracleBackend(model, max_context=qcfg.max_position_embeddings or 8192)
    if backend_name == BACKEND_GPU:
        if not torch.cuda.is_available():
            raise LoadError("the b200 backend needs a CUDA device (use the cpu runtime bundle on hosts without one)")
        if not _supported_on_gpu(cfg):
            raise Unsupported(f"{cfg.architecture.value} (head_dim {cfg.head_dim}) is not served by the sm_100a "
                              "decoder; load it through the cpu-llama provider")
        from ..models.llama import LlamaGpu
        from .kv_pool import PagedKvPool
        from .runner import ModelRunner

        dev = comm.device if comm is not None else torch.device("cuda", torch.cuda.current_device())
        model = LlamaGpu(cfg, comm=comm, device=dev).load_state_dict(weights)
        ctx = min(cfg.max_position_embeddings or 8192, 32768)
        max_batch = 16
        free, _total = torch.cuda.mem_get_info(dev)
        per_block = cfg.num_layers * 2 * model.hkv * 16 * cfg.head_dim * 2
        want = max_batch * ((ctx + 15) // 16) + 64
        nblocks = max(64, min(want, int(free * 0.6) // per_block))
        pool = PagedKvPool(cfg.num_layers, nblocks, model.hkv, cfg.head_dim, 16, device=dev)
        return GpuBackend(ModelRunner(model, pool, max_batch=max_batch, max_seq_len=ctx))
    return OracleBackend(OracleLlama(cfg, weights, dtype=torch.float32, device="cpu"),
                         max_context=cfg.max_position_embeddings or 8192)


# ---- LLaVA: vision tower + projector in front of the same decoder ------------------------------------------------
class LlavaProvider(LlamaProvider):
    """Image-and-text chat over a Hugging Face LLaVA snapshot (the reference's `candle-llava`:
    candle-llm/src/llava.rs:46-693). Every image of the conversation becomes one `<image>` placeholder in its
    message; after tokenisation each placeholder expands to one token per projected patch feature, and the prefill
    replaces those tokens' embeddings by the features."""

    IMAGE_PLACEHOLDER = "<image>"

    def __init__(self, base: LlamaProvider, captioner):
        caps = base._descriptor.capabilities
        caps.supports_vision = True
        super().__init__(base._descriptor, base.backend, base.tokenizer, base.template, base.stop_tokens, base.cfg)
        self.vision = captioner            # media.vision_providers.LlavaCaptioner (tower + projector + token id)

    @staticmethod
    def load(spec: LoadSpec, provider_id: str, backend_name: str, comm=None) -> "LlavaProvider":
        from ..media.vision_providers import LlavaCaptioner
        from ..models.vision import VisionConfig, VisionTower

        p = Path(spec.source)
        top = _read_json(p / "config.json")
        if "vision_config" not in top or "text_config" not in top:
            raise LoadError(f"{p}: not a LLaVA snapshot (config.json lacks vision_config / text_config)")
        w = load_dir(p)
        w = {(k[6:] if k.startswith("model.") and not k.startswith("model.layers") else k): v for k, v in w.items()}
        lmw = {}
        for k, v in w.items():
            if k.startswith("language_model."):
                k2 = k[len("language_model."):]
                lmw[k2 if k2.startswith(("model.", "lm_head.")) else "model." + k2] = v
        if "lm_head.weight" in w:
            lmw["lm_head.weight"] = w["lm_head.weight"]
        cfg = ModelConfig.from_json(top["text_config"])
        tokenizer = Tokenizer.from_file(p / "tokenizer.json")
        tcfg = _read_json(p / "tokenizer_config.json")
        template, thinking, tools = _pick_template(tcfg.get("chat_template") and tcfg, cfg)
        stop = sorted(_eos_ids(top) | _eos_ids(top["text_config"]) |
                      {i for n in _STOP_NAMES if (i := tokenizer.token_to_id(n)) is not None})
        backend = _build_backend(cfg, lmw, backend_name, comm)
        caps = TextLlmCapabilities(max_context_tokens=backend.max_context, max_new_tokens=0, supports_system_prompt=True,
                                   supports_vision=True, supports_video=False, supports_thinking=thinking,
                                   supports_tools=tools, supported_constraints=[Constraint.JSON])
        base = LlamaProvider(TextLlmDescriptor(provider_id, "llava", backend_name, caps), backend, tokenizer, template,
                             stop, cfg)
        on_gpu = backend_name == BACKEND_GPU
        dev, dtype = ("cuda", torch.bfloat16) if on_gpu else ("cpu", torch.float32)
        vcfg = VisionConfig.from_json(top)
        tower = VisionTower(vcfg, {k[len("vision_tower."):]: v for k, v in w.items() if k.startswith("vision_tower.")},
                            dev, dtype)
        proj = {k[len("multi_modal_projector."):]: v.to(dev, dtype) for k, v in w.items()
                if k.startswith("multi_modal_projector.")}
        image_token = int(top.get("image_token_index", top.get("image_token_id", -1)))
        if image_token < 0:
            tid = tokenizer.token_to_id(LlavaProvider.IMAGE_PLACEHOLDER)
            if tid is None:
                raise LoadError(f"{p}: no image token id in config.json and no <image> token in the tokenizer")
            image_token = tid
        cap = LlavaCaptioner(tower, proj, None, tokenizer, image_token, backend_name,
                             int(top.get("vision_feature_layer", -2)),
                             top.get("vision_feature_select_strategy", "default") == "default" and vcfg.kind == "clip")
        return LlavaProvider(base, cap)

    def _render_messages(self, req: TextLlmRequest):
        from ..contracts.core_llm.message import ImageRef, Message, Text

        out = []
        for m in req.messages:
            n = sum(isinstance(c, ImageRef) for c in m.content)
            if n == 0:
                out.append(m)
                continue
            text = (self.IMAGE_PLACEHOLDER + "\n") * n + m.text_content()
            out.append(Message(m.role, [Text(text)], m.thinking, list(m.tool_calls)))
        return out

    def _splice_media(self, req: TextLlmRequest, prompt_ids: list[int]):
        from ..contracts.core_llm.message import ImageRef
        from ..contracts.gen_core.media import Image
        from .backend import set_embed_override

        images = [c for m in req.messages for c in m.content if isinstance(c, ImageRef)]
        if not images:
            return prompt_ids, None
        tid = self.vision.image_token_id
        if prompt_ids.count(tid) != len(images):
            from ..contracts.core_llm import InvalidRequest

            raise InvalidRequest(f"[{self._descriptor.id}] the rendered prompt holds {prompt_ids.count(tid)} image "
                                 f"placeholders for {len(images)} images")
        feats = [self.vision.image_features(Image(i.width, i.height, bytes(i.pixels))) for i in images]
        ids, pos, k = [], [], 0
        for t in prompt_ids:
            if t == tid:
                pos += list(range(len(ids), len(ids) + feats[k].shape[0]))
                ids += [tid] * feats[k].shape[0]
                k += 1
            else:
                ids.append(t)
        seq = self.backend.new_sequence()
        set_embed_override(seq, pos, torch.cat(feats, dim=0))
        return ids, seq


# ---- Qwen3-VL: vision tower with DeepStack in front of the M-RoPE decoder -----------------------------------------
class Qwen3VlProvider(LlamaProvider):
    """Image-and-text chat over a Hugging Face Qwen3-VL snapshot (candle-llm/src/models/qwen35_vision.rs,
    deepstack.rs). Every image becomes `<|vision_start|><|image_pad|><|vision_end|>` in its message; after
    tokenisation the pad token expands to one token per merged patch group, the prefill replaces those embeddings by
    the tower's tokens, uses three-axis positions and adds the DeepStack taps after the first decoder layers. The
    decoder runs on the oracle backend (fp32 on the CPU bundle, bf16 on the device for the b200 bundle): the paged
    sm_100a decoder has no three-axis rotary table."""

    IMAGE_BLOCK = "<|vision_start|><|image_pad|><|vision_end|>"

    def __init__(self, base: LlamaProvider, tower, image_token_id: int, video_token_id: int | None = None):
        caps = base._descriptor.capabilities
        caps.supports_vision = True
        caps.supports_video = video_token_id is not None
        super().__init__(base._descriptor, base.backend, base.tokenizer, base.template, base.stop_tokens, base.cfg)
        self.tower, self.image_token_id, self.video_token_id = tower, image_token_id, video_token_id

    @staticmethod
    def load(spec: LoadSpec, provider_id: str, backend_name: str, comm=None) -> "Qwen3VlProvider":
        from ..models.qwen3_vl import Qwen3VlVisionConfig, Qwen3VlVisionTower

        p = Path(spec.source)
        top = _read_json(p / "config.json")
        if "vision_config" not in top or "text_config" not in top:
            raise LoadError(f"{p}: not a Qwen3-VL snapshot (config.json lacks vision_config / text_config)")
        w = load_dir(p)
        text = {k.replace("model.language_model.", "model."): v for k, v in w.items()
                if not k.startswith(("model.visual.", "visual."))}
        cfg = ModelConfig.from_json(top)
        tokenizer = Tokenizer.from_file(p / "tokenizer.json")
        tcfg = _read_json(p / "tokenizer_config.json")
        template, thinking, tools = _pick_template(tcfg.get("chat_template") and tcfg, cfg)
        stop = sorted(_eos_ids(top) | _eos_ids(top["text_config"]) |
                      {i for n in _STOP_NAMES if (i := tokenizer.token_to_id(n)) is not None})
        on_gpu = backend_name == BACKEND_GPU
        if on_gpu and not torch.cuda.is_available():
            raise LoadError("the b200 backend needs a CUDA device (use the cpu runtime bundle on hosts without one)")
        dev, dtype = ("cuda", torch.bfloat16) if on_gpu else ("cpu", torch.float32)
        if on_gpu and _supported_on_gpu(cfg) and os.environ.get("SWB_QWEN3_VL_DECODER", "paged") != "oracle":
            # the paged sm_100a decoder: per-token three-axis rotary table and DeepStack taps ride on the prefill step
            backend = _build_backend(cfg, text, backend_name, comm)
        else:
            backend = OracleBackend(OracleLlama(cfg, text, dtype=dtype, device=dev),
                                    max_context=cfg.max_position_embeddings or 8192)
        caps = TextLlmCapabilities(max_context_tokens=backend.max_context, max_new_tokens=0, supports_system_prompt=True,
                                   supports_vision=True, supports_video=False, supports_thinking=thinking,
                                   supports_tools=tools, supported_constraints=[Constraint.JSON])
        base = LlamaProvider(TextLlmDescriptor(provider_id, "qwen3-vl", backend_name, caps), backend, tokenizer, template,
                             stop, cfg)
        prefix = "model.visual." if any(k.startswith("model.visual.") for k in w) else "visual."
        tower = Qwen3VlVisionTower(Qwen3VlVisionConfig.from_json(top), w, dev, dtype, prefix=prefix)
        image_token = top.get("image_token_id")
        if image_token is None:
            image_token = tokenizer.token_to_id("<|image_pad|>")
        if image_token is None:
            raise LoadError(f"{p}: no image_token_id in config.json and no <|image_pad|> token in the tokenizer")
        video_token = top.get("video_token_id")
        if video_token is None:
            video_token = tokenizer.token_to_id("<|video_pad|>")
        return Qwen3VlProvider(base, tower, int(image_token), int(video_token) if video_token is not None else None)

    def _render_messages(self, req: TextLlmRequest):
        """Images become one vision block each; a video becomes one block per temporal patch (two frames), each
        announced by the patch's time in seconds."""
        from ..contracts.core_llm.message import ImageRef, Message, Text, VideoRef
        from ..models.qwen3_vl import video_placeholder_text

        T = self.tower.cfg.temporal_patch_size
        out = []
        for m in req.messages:
            blocks = ""
            for c in m.content:
                if isinstance(c, ImageRef):
                    blocks += self.IMAGE_BLOCK
                elif isinstance(c, VideoRef):
                    ts = list(c.timestamps)
                    while len(ts) % T:
                        ts.append(ts[-1])
                    blocks += video_placeholder_text([sum(ts[i:i + T]) / T for i in range(0, len(ts), T)])
            if not blocks:
                out.append(m)
                continue
            out.append(Message(m.role, [Text(blocks + m.text_content())], m.thinking, list(m.tool_calls)))
        return out

    def _splice_media(self, req: TextLlmRequest, prompt_ids: list[int]):
        import numpy as np

        from ..contracts.core_llm import InvalidRequest
        from ..contracts.core_llm.message import ImageRef, VideoRef
        from ..models.qwen3_vl import image_to_patches, mrope_positions, video_to_patches
        from .backend import set_embed_override, set_mrope_override

        media = [c for m in req.messages for c in m.content if isinstance(c, (ImageRef, VideoRef))]
        if not media:
            return prompt_ids, None
        vc = self.tower.cfg
        rgb = lambda im: torch.from_numpy(np.frombuffer(bytes(im.pixels), dtype=np.uint8)                  # noqa: E731
                                          .reshape(im.height, im.width, 3).copy())
        patches, tower_grids, runs = [], [], []          # runs: one (placeholder id, (1, h, w)) per vision run of the prompt
        for c in media:
            if isinstance(c, ImageRef):
                pt, g = image_to_patches(rgb(c), vc)
                runs.append((self.image_token_id, g))
            else:
                if self.video_token_id is None:
                    raise InvalidRequest(f"[{self._descriptor.id}] this snapshot has no video placeholder token")
                pt, g, _ = video_to_patches([rgb(f) for f in c.frames], list(c.timestamps), vc)
                runs += [(self.video_token_id, (1, g[1], g[2]))] * g[0]
            patches.append(pt)
            tower_grids.append(g)
        vision_ids = {self.image_token_id} | ({self.video_token_id} if self.video_token_id is not None else set())
        found = [t for t in prompt_ids if t in vision_ids]
        if found != [tid for tid, _ in runs]:
            raise InvalidRequest(f"[{self._descriptor.id}] the rendered prompt holds {len(found)} vision placeholders for "
                                 f"{len(runs)} vision runs")
        tokens, taps = self.tower.forward(torch.cat(patches, 0), tower_grids)
        m2 = vc.spatial_merge_size ** 2
        ids, rows, k = [], [], 0
        for t in prompt_ids:
            if t in vision_ids:
                n = runs[k][1][1] * runs[k][1][2] // m2
                rows += list(range(len(ids), len(ids) + n))
                ids += [t] * n
                k += 1
            else:
                ids.append(t)
        pos, nxt = mrope_positions(ids, [g for _, g in runs], vision_ids, vc.spatial_merge_size)
        seq = self.backend.new_sequence()
        set_embed_override(seq, rows, tokens)
        set_mrope_override(seq, pos, nxt, torch.tensor(rows), taps)
        return ids, seq


def _can_load_qwen3_vl(spec: LoadSpec) -> bool:
    p = Path(spec.source)
    top = _read_json(p / "config.json") if p.is_dir() else {}
    return "vision_config" in top and "text_config" in top and "qwen3_vl" in str(top.get("model_type", "")).lower()


def _can_load_llava(spec: LoadSpec) -> bool:
    p = Path(spec.source)
    top = _read_json(p / "config.json") if p.is_dir() else {}
    return "vision_config" in top and "text_config" in top and "llava" in str(top.get("model_type", "")).lower()


# ---- registrations ------------------------------------------------------------------------------------------
def _descriptor(pid: str, backend: str) -> TextLlmDescriptor:
    return TextLlmDescriptor(pid, "llama", backend, TextLlmCapabilities(
        max_context_tokens=0, max_new_tokens=0, supports_system_prompt=True, supports_vision=False,
        supports_video=False, supports_thinking=False, supports_tools=False, supported_constraints=[Constraint.JSON]))


def _descriptor_vision(pid: str, backend: str) -> TextLlmDescriptor:
    d = _descriptor(pid, backend)
    d.family = "llava"
    d.capabilities.supports_vision = True
    return d


def _can_load_gpu(spec: LoadSpec) -> bool:
    if _can_load_qwen3_vl(spec):            # a snapshot with a vision tower belongs to the vision-language provider
        return False
    cfg = probe_config(spec)
    return cfg is not None and (_supported_on_gpu(cfg) or cfg.architecture is Architecture.QWEN35)


def _can_load_cpu(spec: LoadSpec) -> bool:
    return not _can_load_qwen3_vl(spec) and probe_config(spec) is not None


B200_LLAVA = TextLlmRegistration(lambda: _descriptor_vision("b200-llava", BACKEND_GPU),
                                 lambda spec: LlavaProvider.load(spec, "b200-llava", BACKEND_GPU), _can_load_llava)
CPU_LLAVA = TextLlmRegistration(lambda: _descriptor_vision("cpu-llava", BACKEND_CPU),
                                lambda spec: LlavaProvider.load(spec, "cpu-llava", BACKEND_CPU), _can_load_llava)
def _descriptor_qwen3_vl(pid: str, backend: str) -> TextLlmDescriptor:
    d = _descriptor_vision(pid, backend)
    d.family = "qwen3-vl"
    return d


B200_QWEN3_VL = TextLlmRegistration(lambda: _descriptor_qwen3_vl("b200-qwen3-vl", BACKEND_GPU),
                                    lambda spec: Qwen3VlProvider.load(spec, "b200-qwen3-vl", BACKEND_GPU), _can_load_qwen3_vl)
CPU_QWEN3_VL = TextLlmRegistration(lambda: _descriptor_qwen3_vl("cpu-qwen3-vl", BACKEND_CPU),
                                   lambda spec: Qwen3VlProvider.load(spec, "cpu-qwen3-vl", BACKEND_CPU), _can_load_qwen3_vl)
B200_LLAMA = TextLlmRegistration(lambda: _descriptor("b200-llama", BACKEND_GPU),
                                 lambda spec: LlamaProvider.load(spec, "b200-llama", BACKEND_GPU), _can_load_gpu)
CPU_LLAMA = TextLlmRegistration(lambda: _descriptor("cpu-llama", BACKEND_CPU),
                                lambda spec: LlamaProvider.load(spec, "cpu-llama", BACKEND_CPU), _can_load_cpu)
