"""Tiny random-weight snapshots written to disk so providers are exercised through their real load path
(the reference's T3 tier: candle-llm/tests/conformance.rs writes a 2-layer random snapshot + WordLevel tokenizer)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from ..io import gguf as gguf_io
from ..io import gguf_quants as gq
from ..io.safetensors_io import save_file
from ..models.config import ModelConfig
from ..models.oracle import random_llama_weights

WORDS = ["<unk>", "<|begin_of_text|>", "<|eot_id|>", "<|start_header_id|>", "<|end_header_id|>", "system", "user",
         "assistant", "hello", "world", "the", "a", "cat", "dog", "sat", "on", "mat", "{", "}", "\"", ":", ",", "1",
         "2", "3", "true", "null", "yes", "no", "ok", "<think>", "</think>"]


def wordlevel_tokenizer_json(vocab_size: int) -> str:
    words = list(WORDS)
    while len(words) < vocab_size:
        words.append(f"w{len(words)}")
    vocab = {w: i for i, w in enumerate(words[:vocab_size])}
    added = [{"id": vocab[w], "content": w, "single_word": False, "lstrip": False, "rstrip": False,
              "normalized": False, "special": True}
             for w in ("<|begin_of_text|>", "<|eot_id|>", "<|start_header_id|>", "<|end_header_id|>") if w in vocab]
    return json.dumps({"version": "1.0", "truncation": None, "padding": None, "added_tokens": added,
                       "normalizer": None, "pre_tokenizer": {"type": "WhitespaceSplit"}, "post_processor": None,
                       "decoder": {"type": "Fuse"} if False else None,
                       "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "<unk>"}})


def tiny_config(head_dim: int = 8, hidden: int = 32, layers: int = 2, vocab: int = 64, model_type: str = "llama",
                **extra) -> dict:
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": model_type, "hidden_size": hidden,
           "intermediate_size": hidden * 2, "num_hidden_layers": layers, "num_attention_heads": 4,
           "num_key_value_heads": 2, "head_dim": head_dim, "vocab_size": vocab, "rms_norm_eps": 1e-5,
           "rope_theta": 10000.0, "tie_word_embeddings": True, "max_position_embeddings": 256, "eos_token_id": 2}
    cfg.update(extra)
    return cfg


def write_snapshot(directory: str | Path, cfg_json: dict | None = None, seed: int = 0, std: float = 0.3,
                   chat_template: str | None = None, dtype: torch.dtype = torch.float32) -> Path:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    cfg_json = cfg_json or tiny_config()
    cfg = ModelConfig.from_json(cfg_json)
    weights = random_llama_weights(cfg, seed=seed, std=std, dtype=dtype)
    save_file(weights, d / "model.safetensors", {"format": "pt"})
    (d / "config.json").write_text(json.dumps(cfg_json))
    (d / "tokenizer.json").write_text(wordlevel_tokenizer_json(cfg.vocab_size))
    tcfg = {"bos_token": "<|begin_of_text|>", "eos_token": "<|eot_id|>"}
    if chat_template is not None:
        tcfg["chat_template"] = chat_template
    (d / "tokenizer_config.json").write_text(json.dumps(tcfg))
    return d


def write_gguf_from_snapshot(snapshot: str | Path, path: str | Path, quant: str = "Q8_0") -> Path:
    """Packs a snapshot's tensors into a GGUF file (2-D weights in `quant`, 1-D in F32, llama q/k permuted)."""
    from ..io.safetensors_io import load_dir

    snap = Path(snapshot)
    cfg_json = json.loads((snap / "config.json").read_text())
    cfg = ModelConfig.from_json(cfg_json)
    inv = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
           "lm_head.weight": "output.weight"}
    layer_inv = {v: k for k, v in gguf_io._LAYER_MAP.items()}
    tensors = {}
    for name, t in load_dir(snap).items():
        t = t.float()
        if name in inv:
            g = inv[name]
        else:
            parts = name.split(".")
            key = ".".join(parts[3:-1])
            g = f"blk.{parts[2]}.{layer_inv[key]}.{parts[-1]}"
        if name.endswith("self_attn.q_proj.weight"):
            t = gguf_io.permute_qk(t, cfg.num_heads)
        elif name.endswith("self_attn.k_proj.weight"):
            t = gguf_io.permute_qk(t, cfg.num_kv_heads)
        x = t.contiguous().numpy()
        block = gq.BLOCK[quant][1]
        if t.dim() == 2 and t.shape[1] % block == 0:
            raw = gq.quantize_q8_0(x) if quant == "Q8_0" else gq.quantize_q4_k(x)
            tensors[g] = (raw, quant, tuple(t.shape))
        else:
            tensors[g] = (x.astype(np.float32).view(np.uint8).reshape(-1), "F32", tuple(t.shape))
    a = "llama"
    md = {"general.architecture": a, "general.alignment": 32, f"{a}.embedding_length": cfg.hidden_size,
          f"{a}.block_count": cfg.num_layers, f"{a}.feed_forward_length": cfg.intermediate_size,
          f"{a}.attention.head_count": cfg.num_heads, f"{a}.attention.head_count_kv": cfg.num_kv_heads,
          f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), f"{a}.rope.freq_base": float(cfg.rope_theta),
          f"{a}.context_length": cfg.max_position_embeddings or 256, f"{a}.attention.key_length": cfg.head_dim,
          "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": [f"t{i}" for i in range(cfg.vocab_size)],
          "tokenizer.ggml.merges": [], "tokenizer.ggml.token_type": [1] * cfg.vocab_size,
          "tokenizer.ggml.eos_token_id": 2}
    gguf_io.write_gguf(path, md, tensors)
    return Path(path)
