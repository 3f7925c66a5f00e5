"""Public batched-generation API over the model runner (the call an application makes).

`LlmEngine.generate_batch` is the synchronous batched decode of the reference's `generate_batch`
(candle-llm/src/decode/batch.rs:54-283) re-designed for paged KV: no left padding, no additive masks —
each sequence owns a block table, prompts are prefilled as one ragged batch (in waves bounded by a token
budget), and rows retire independently.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import torch

from ..models.llama import LlamaGpu
from .kv_pool import PagedKvPool, PagedSequence
from .runner import ModelRunner


@dataclass
class BatchResult:
    tokens: list[list[int]]
    finish_reasons: list[str]
    prefill_ms: float = 0.0
    steps: int = 0


@dataclass
class EngineConfig:
    block_size: int = 16
    max_batch: int = 64
    max_seq_len: int = 8192
    prefill_token_budget: int = 16384   # tokens per prefill forward (bounds activation memory)
    kv_bytes: int | None = None          # None: size the pool for max_batch * max_seq_len tokens
    use_graphs: bool = True


class LlmEngine:
    def __init__(self, model: LlamaGpu, cfg: EngineConfig | None = None):
        self.model = model
        self.cfg = cfg or EngineConfig()
        c, m = self.cfg, model.cfg
        if c.kv_bytes is not None:
            nblocks = PagedKvPool.blocks_for_budget(c.kv_bytes, m.num_layers, model.hkv, m.head_dim, c.block_size)
        else:
            nblocks = c.max_batch * ((c.max_seq_len + c.block_size - 1) // c.block_size) + 8
        if hasattr(model, "make_pool"):      # pipeline-sharded model: one KV tensor per stage device, shared block ids
            self.pool = model.make_pool(nblocks, c.block_size)
        else:
            self.pool = PagedKvPool(m.num_layers, nblocks, model.hkv, m.head_dim, c.block_size, device=model.device)
        self.runner = ModelRunner(model, self.pool, max_batch=c.max_batch, max_seq_len=c.max_seq_len,
                                  use_graphs=c.use_graphs)

    def new_sequence(self) -> PagedSequence:
        return PagedSequence(self.pool)

    def prefill_batch(self, seqs: list[PagedSequence], prompts: list[list[int]]) -> list[int]:
        """Ragged prefill in waves under the token budget; returns each sequence's first greedy token."""
        first: list[int] = [0] * len(seqs)
        i = 0
        while i < len(seqs):
            j, tok = i, 0
            while j < len(seqs) and (j == i or tok + len(prompts[j]) <= self.cfg.prefill_token_budget):
                tok += len(prompts[j])
                j += 1
            out = self.runner.prefill(seqs[i:j], prompts[i:j])
            for k, t in enumerate(out.tolist()):
                first[i + k] = int(t)
            i = j
        return first

    def generate_batch(self, prompts: list[list[int]], max_new_tokens: int, stop_tokens: tuple[int, ...] = (),
                       on_step: Callable[[int, list[int]], None] | None = None) -> BatchResult:
        """Greedy batched generation; every step's tokens reach the host (streaming granularity)."""
        seqs = [self.new_sequence() for _ in prompts]
        try:
            toks = self.prefill_batch(seqs, prompts)
            outs: list[list[int]] = [[] for _ in prompts]
            reasons = ["length"] * len(prompts)
            live = list(range(len(prompts)))
            steps = 0
            while live and steps < max_new_tokens:
                nxt_live = []
                for i in live:
                    if toks[i] in stop_tokens:
                        reasons[i] = "stop"
                    else:
                        outs[i].append(toks[i])
                        if len(outs[i]) < max_new_tokens:
                            nxt_live.append(i)
                if on_step is not None:
                    on_step(steps, [toks[i] for i in live])
                live = nxt_live
                steps += 1
                if not live:
                    break
                new = self.runner.decode([seqs[i] for i in live], [toks[i] for i in live])
                for k, i in enumerate(live):
                    toks[i] = int(new[k])
            return BatchResult(outs, reasons, steps=steps)
        finally:
            for s in seqs:
                s.release()
