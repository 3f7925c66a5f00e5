"""Snapshot preparation: convert a checkpoint once into a self-contained HF-layout directory that loads fast.

Parity: candle-llm/src/prepare.rs:63-360. An HF snapshot is passed through (dense) or has its projection
weights quantise-rounded (Q4 -> Q4_K, Q8 -> Q8_0 numerics) with `quantization{bits}` stamped into config.json; a
GGUF file is dequantised to an f16 HF snapshot with config.json, tokenizer.json and the chat template rebuilt
from its metadata."""
from __future__ import annotations

import json
import shutil
from pathlib import Path

import torch

from ..contracts.core_llm import (ModelFormat, PrepareReport, PrepareSpec, SnapshotPreparerRegistration, Unsupported,
                                  detect_format)
from ..contracts.errors import LoadError
from . import gguf as gguf_io
from .safetensors_io import iter_dir, save_file

_SIDE_FILES = ("tokenizer.json", "tokenizer_config.json", "generation_config.json", "special_tokens_map.json",
               "chat_template.jinja", "tokenizer.model", "vocab.json", "merges.txt")
_PROJ = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "gate_proj.weight", "up_proj.weight",
         "down_proj.weight", "qkv_proj.weight", "gate_up_proj.weight")


def can_prepare(spec: PrepareSpec) -> bool:
    try:
        fmt = detect_format(spec.source)
    except Exception:
        return False
    if fmt is ModelFormat.GGUF:
        p = Path(spec.source)
        if p.is_dir():
            ggufs = sorted(p.glob("*.gguf"))
            p = ggufs[0] if ggufs else p
        return gguf_io.gguf_architecture(p) in gguf_io.ARCH_TO_HF
    return True


def prepare_hf(spec: PrepareSpec) -> PrepareReport:
    from ..engine.provider import quantize_roundtrip

    src, out = Path(spec.source), Path(spec.out_dir)
    if src.is_file():
        raise Unsupported(f"'{src}': a bare .safetensors file has no config.json; pass the snapshot directory")
    out.mkdir(parents=True, exist_ok=True)
    cfg = json.loads((src / "config.json").read_text())
    bits = spec.quantize.value if spec.quantize is not None else None
    tensors, n = {}, 0
    for name, t in iter_dir(src):
        if bits is not None and name.endswith(_PROJ) and t.dim() == 2:
            t = quantize_roundtrip(t.float(), bits).to(t.dtype)
        tensors[name] = t
        n += 1
    save_file(tensors, out / "model.safetensors", {"format": "pt"})
    if bits is not None:
        cfg["quantization"] = {"bits": bits}
    (out / "config.json").write_text(json.dumps(cfg, indent=2))
    for f in _SIDE_FILES:
        if (src / f).is_file():
            shutil.copyfile(src / f, out / f)
    return PrepareReport(ModelFormat.SAFETENSORS, spec.quantize, out, n, passthrough=bits is None)


def prepare_gguf(spec: PrepareSpec) -> PrepareReport:
    from ..engine.provider import quantize_roundtrip

    src, out = Path(spec.source), Path(spec.out_dir)
    if src.is_dir():
        ggufs = sorted(src.glob("*.gguf"))
        if not ggufs:
            raise LoadError(f"no *.gguf under {src}")
        src = ggufs[0]
    ck = gguf_io.GgufCheckpoint(src)
    out.mkdir(parents=True, exist_ok=True)
    cfg = ck.config()
    bits = spec.quantize.value if spec.quantize is not None else None
    tensors = {}
    for name, t in ck.tensors(torch.float32).items():
        if bits is not None and name.endswith(_PROJ) and t.dim() == 2:
            t = quantize_roundtrip(t, bits)
        tensors[name] = t.to(torch.float16)
    save_file(tensors, out / "model.safetensors", {"format": "pt"})
    if bits is not None:
        cfg["quantization"] = {"bits": bits}
    cfg["torch_dtype"] = "float16"
    (out / "config.json").write_text(json.dumps(cfg, indent=2))
    tj = ck.tokenizer_json()
    if tj is not None:
        (out / "tokenizer.json").write_text(tj)
    tcfg = {}
    if ck.chat_template():
        tcfg["chat_template"] = ck.chat_template()
    toks = ck.file.metadata.get("tokenizer.ggml.tokens") or []
    for key, name in (("tokenizer.ggml.bos_token_id", "bos_token"), ("tokenizer.ggml.eos_token_id", "eos_token")):
        i = ck.file.metadata.get(key)
        if isinstance(i, int) and 0 <= i < len(toks):
            tcfg[name] = toks[i]
    (out / "tokenizer_config.json").write_text(json.dumps(tcfg, indent=2))
    n = len(tensors)
    ck.file.close()
    return PrepareReport(ModelFormat.GGUF, spec.quantize, out, n, passthrough=False)


def prepare(spec: PrepareSpec) -> PrepareReport:
    fmt = detect_format(spec.source)
    return prepare_gguf(spec) if fmt is ModelFormat.GGUF else prepare_hf(spec)


def registration(backend: str) -> SnapshotPreparerRegistration:
    return SnapshotPreparerRegistration(lambda: backend, can_prepare, prepare)
