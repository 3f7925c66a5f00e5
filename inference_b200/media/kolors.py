"""Kolors text-to-image provider `kolors` (and `cpu_kolors` on the fp32 backend)
(parity: candle-gen-kolors/src/lib.rs, pipeline.rs, chatglm3.rs, tokenizer.rs, sampler.rs, config.rs).

Kolors is the SDXL UNet and autoencoder with a ChatGLM3-6B prompt encoder in place of the two CLIPs: the input of
ChatGLM3's last layer (256 left-padded positions, 4096 wide) is projected to the UNet's 2048-wide cross-attention
context, the last layer's state at the final token (4096) replaces the pooled CLIP vector (so the additional embedding
reads 4096 + 6 * 256 = 5632 numbers). Sampling is noise prediction over an 1100-step scaled-linear table
(betas 0.00085 .. 0.014), Euler by default, 50 steps, classifier-free guidance 5.

Snapshot layout (diffusers): `unet/`, `text_encoder/` (ChatGLM3: config.json + weights) + `tokenizer/tokenizer.model`,
`vae/`; `swb_config.json` overrides dimensions for synthetic snapshots."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable

import torch

from ..contracts.errors import LoadError, Unsupported
from ..contracts.gen_core.generator import Capabilities, Modality, ModelDescriptor
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import AdapterKind, LoadSpec
from ..contracts.gen_core.sampling import SCHEDULERS, SOLVERS, DiscreteModelSampling
from ..contracts.gen_core.sampling.policy import AlphaSchedule
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.unet_sdxl import SdxlUnetConfig
from .sdxl import SdxlConditioning, SdxlGenerator, SdxlPipeline

MODEL_ID = "kolors"
TRAIN_TIMESTEPS, BETA_START, BETA_END = 1100, 0.00085, 0.014
CONTEXT_DIM = 4096


class ChatGlmConditioner:
    def __init__(self, encoder):
        self.encoder = encoder

    def encode(self, prompt: str) -> SdxlConditioning:
        context, pooled = self.encoder.encode(prompt)
        return SdxlConditioning(context, pooled)


class KolorsPipeline(SdxlPipeline):
    model_id, default_steps, default_guidance = MODEL_ID, 50, 5.0
    default_sampler, default_scheduler = "euler", "normal"

    @staticmethod
    def default_unet_config() -> SdxlUnetConfig:
        return SdxlUnetConfig(projection_class_embeddings_input_dim=CONTEXT_DIM + 6 * 256, encoder_hid_dim=CONTEXT_DIM)

    @staticmethod
    def model_sampling() -> DiscreteModelSampling:
        return DiscreteModelSampling(schedule=AlphaSchedule.scaled_linear(TRAIN_TIMESTEPS, BETA_START, BETA_END))

    def load_text(self):
        if self.text_kind == "hash":
            from .sdxl import HashDualEncoders

            c = self.unet_cfg
            return HashDualEncoders(c.encoder_hid_dim or c.cross_attention_dim,
                                    c.projection_class_embeddings_input_dim - 6 * c.addition_time_embed_dim, self.device, self.dtype)
        import sentencepiece as spm

        from ..io.safetensors_io import load_dir
        from ..models.chatglm3 import ChatGlm3PromptEncoder

        te, tk = self.root / "text_encoder", self.root / "tokenizer" / "tokenizer.model"
        if not (te / "config.json").is_file() or not tk.exists():
            raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks text_encoder/config.json or tokenizer/tokenizer.model")
        files = sorted(te.glob("*.safetensors"))
        if files:
            weights = load_dir(te)
        else:
            weights = {}
            for f in sorted(te.glob("pytorch_model*.bin")):
                weights.update(torch.load(f, map_location="cpu", weights_only=True))
            if not weights:
                raise LoadError(f"{MODEL_ID}: {te} holds no *.safetensors or pytorch_model*.bin weights")
        enc = ChatGlm3PromptEncoder(json.loads((te / "config.json").read_text()), weights,
                                    spm.SentencePieceProcessor(model_file=str(tk)), self.device, self.dtype)
        return ChatGlmConditioner(enc)


def kolors_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family="kolors", backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False, conditioning=[],
            supports_lora=True, supports_lokr=False, samplers=list(SOLVERS), schedulers=list(SCHEDULERS),
            supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8, supports_sequential_offload=True),
        required_components=[])


def _load(backend: str, prefix: str) -> Callable[[LoadSpec], SdxlGenerator]:
    def load(spec: LoadSpec) -> SdxlGenerator:
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
        pipe = KolorsPipeline(Path(spec.weights.path), backend, device)
        pipe.adapters = list(spec.adapters)
        return SdxlGenerator(pipe, kolors_descriptor(backend, prefix), spec.offload_policy)
    return load


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=lambda: kolors_descriptor(backend, prefix), load=_load(backend, prefix))]


def write_synthetic_snapshot(root, seed: int = 0, text: str = "hash") -> Path:
    """A tiny random Kolors-shaped snapshot. text="chatglm" also writes a 3-layer random ChatGLM3-named encoder and a
    toy SentencePiece model."""
    from ..io.safetensors_io import save_file
    from ..models.unet_sdxl import random_sdxl_unet_weights
    from ..models.vae import VaeConfig, random_vae_weights
    from .chroma import native_vae_to_diffusers
    from .sdxl import VAE_SCALE

    root = Path(root)
    hid = 64
    unet = SdxlUnetConfig(block_out_channels=(32, 64, 128), transformer_layers_per_block=(0, 1, 2), attention_head_dim=64,
                          cross_attention_dim=48, addition_time_embed_dim=8, projection_class_embeddings_input_dim=hid + 48,
                          norm_groups=8, encoder_hid_dim=hid)
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1, z_channels=4, scale_factor=VAE_SCALE, shift_factor=0.0)
    (root / "unet").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_sdxl_unet_weights(unet, seed).items()},
              root / "unet" / "diffusion_pytorch_model.safetensors")
    save_file({k: v.bfloat16() for k, v in native_vae_to_diffusers(random_vae_weights(vae, seed + 1), len(vae.ch_mult)).items()},
              root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "unet": {"block_out_channels": list(unet.block_out_channels),
                 "transformer_layers_per_block": list(unet.transformer_layers_per_block),
                 "attention_head_dim": unet.attention_head_dim, "cross_attention_dim": unet.cross_attention_dim,
                 "addition_time_embed_dim": unet.addition_time_embed_dim,
                 "projection_class_embeddings_input_dim": unet.projection_class_embeddings_input_dim,
                 "norm_groups": unet.norm_groups, "encoder_hid_dim": hid},
        "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks}, "text": text}))
    if text == "chatglm":
        import io

        import sentencepiece as spm

        from ..models.chatglm3 import chatglm_from_glm_weights, glm_config_from_chatglm
        from ..models.oracle import random_llama_weights

        (root / "tokenizer").mkdir(exist_ok=True)
        corpus = ["a red fox jumps over the lazy dog", "a lighthouse at dusk in an oil painting", "blurry low quality picture",
                  "the quick brown fox and the slow green turtle", "mountains rivers forests and deserts at night"] * 4
        model = io.BytesIO()
        spm.SentencePieceTrainer.train(sentence_iterator=iter(corpus), model_writer=model, vocab_size=60, model_type="bpe",
                                       character_coverage=1.0, hard_vocab_limit=False)
        (root / "tokenizer" / "tokenizer.model").write_bytes(model.getvalue())
        n_words = spm.SentencePieceProcessor(model_proto=model.getvalue()).vocab_size()
        cj = {"num_layers": 3, "hidden_size": hid, "ffn_hidden_size": 96, "num_attention_heads": 4, "multi_query_attention": True,
              "multi_query_group_num": 2, "kv_channels": 16, "padded_vocab_size": n_words + 8, "layernorm_epsilon": 1e-5,
              "seq_length": 512}
        (root / "text_encoder").mkdir(exist_ok=True)
        (root / "text_encoder" / "config.json").write_text(json.dumps(cj))
        cfg = glm_config_from_chatglm(cj)
        w = random_llama_weights(cfg, seed + 2, std=0.08, bias=True)
        save_file({k: v.bfloat16().contiguous() for k, v in chatglm_from_glm_weights(w, cfg).items()},
                  root / "text_encoder" / "model.safetensors")
    return root
