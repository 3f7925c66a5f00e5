"""T5-XXL encoder + CLIP-L text encoder loading for FLUX snapshots (`text_encoder/` = CLIP, `text_encoder_2/` = T5,
`tokenizer/`, `tokenizer_2/`; parity: candle-gen-flux/src/pipeline.rs:552-620,1011-1051)."""
from __future__ import annotations

from pathlib import Path

from ..contracts.errors import LoadError


def load_t5_clip(root: Path, backend: str, device):
    root = Path(root)
    missing = [d for d in ("text_encoder", "text_encoder_2", "tokenizer", "tokenizer_2") if not (root / d).is_dir()]
    if missing:
        raise LoadError(f"flux snapshot {root}: missing text-encoder components {missing}")
    from .text_models import T5ClipEncoders

    return T5ClipEncoders.from_snapshot(root, backend, device)
