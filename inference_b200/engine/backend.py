"""Backend-neutral decode interface the generation loops are written against.

Two implementations: `GpuBackend` (sm_100a model runner over the paged KV pool) and `OracleBackend` (the fp32
PyTorch oracle with contiguous caches, used by the CPU runtime and as the parity reference). The reference's
`Decode` trait (candle-llm/src/decode/stream.rs:21-31) steps one contiguous cache; here a step takes any set of
sequences with any number of new tokens each, which covers prefill, chunked prefill, decode, batched decode
and speculative verify with one call."""
from __future__ import annotations

from typing import Any, Protocol

import torch

from ..models.oracle import ContiguousKvCache, OracleLlama
from .kv_pool import PagedSequence
from .runner import ModelRunner


class DecodeBackend(Protocol):
    vocab_size: int
    max_context: int

    def new_sequence(self) -> Any: ...
    def length(self, seq: Any) -> int: ...
    def forward(self, seqs: list[Any], new_tokens: list[list[int]], all_positions: bool = False) -> list[torch.Tensor]:
        """Appends new_tokens[i] to seqs[i]; returns per-sequence fp32 logits on the host-visible device:
        [vocab] (last position) or [len_i, vocab] when all_positions."""
    def forward_greedy(self, seqs: list[Any], new_tokens: list[list[int]]) -> list[int]: ...
    def truncate(self, seq: Any, length: int) -> None: ...
    def fork(self, seq: Any, n_tokens: int) -> Any:
        """A new sequence sharing the first n_tokens tokens of seq's cache (copy-on-write where supported)."""
    def release(self, seq: Any) -> None: ...


def set_embed_override(seq: Any, positions: list[int], values: torch.Tensor) -> None:
    """Vision-language prompts: the next forward that appends tokens to `seq` replaces the embeddings of the new
    tokens at `positions` (indices within that call's token list) by `values` [len(positions), hidden]."""
    seq.pending_embeds = (list(positions), values)


def set_mrope_override(seq: Any, positions: torch.Tensor, next_position: int, rows: torch.Tensor,
                       taps: list[torch.Tensor]) -> None:
    """Qwen3-VL prompts: the next forward on `seq` uses the three-axis positions [3, S] of its new tokens and adds the
    DeepStack taps at `rows`; later tokens continue at `next_position`."""
    seq.pending_mrope = (positions, int(next_position), rows, taps)


def _take_mrope(seqs) -> list | None:
    mr = [getattr(s, "pending_mrope", None) for s in seqs]
    if not any(m is not None for m in mr):
        return None
    for s in seqs:
        if getattr(s, "pending_mrope", None) is not None:
            s.pending_mrope = None
    return mr


def _take_overrides(seqs) -> list | None:
    ov = [getattr(s, "pending_embeds", None) for s in seqs]
    if not any(o is not None for o in ov):
        return None
    for s in seqs:
        if getattr(s, "pending_embeds", None) is not None:
            s.pending_embeds = None
    return ov


class GpuBackend:
    def __init__(self, runner: ModelRunner):
        self.runner = runner
        self.vocab_size = runner.model.cfg.vocab_size
        self.max_context = runner.max_seq_len

    def new_sequence(self) -> PagedSequence:
        return PagedSequence(self.runner.pool)

    def length(self, seq: PagedSequence) -> int:
        return seq.length

    def _is_decode(self, seqs, new_tokens) -> bool:
        return all(len(t) == 1 for t in new_tokens) and len(seqs) <= self.runner.max_batch

    def forward(self, seqs, new_tokens, all_positions=False):
        ov, mr = _take_overrides(seqs), _take_mrope(seqs)
        if ov is None and mr is None and not all_positions and self._is_decode(seqs, new_tokens):
            logits = self.runner.decode(seqs, [t[0] for t in new_tokens], want_logits=True)
            return [logits[i] for i in range(len(seqs))]
        logits = self.runner.prefill(seqs, new_tokens, want_logits=True, all_positions=all_positions,
                                     embed_overrides=ov, mrope_overrides=mr)
        if not all_positions:
            return [logits[i] for i in range(len(seqs))]
        out, o = [], 0
        for t in new_tokens:
            out.append(logits[o:o + len(t)])
            o += len(t)
        return out

    def forward_greedy(self, seqs, new_tokens):
        ov, mr = _take_overrides(seqs), _take_mrope(seqs)
        if ov is None and mr is None and self._is_decode(seqs, new_tokens):
            return [int(x) for x in self.runner.decode(seqs, [t[0] for t in new_tokens]).tolist()]
        return [int(x) for x in self.runner.prefill(seqs, new_tokens, embed_overrides=ov, mrope_overrides=mr).tolist()]

    def truncate(self, seq, length):
        seq.truncate(length)

    def fork(self, seq, n_tokens):
        bs = self.runner.pool.block_size
        whole = (n_tokens // bs) * bs
        f = PagedSequence.seeded(self.runner.pool, seq.shareable_prefix_blocks(whole), whole)
        if getattr(seq, "rope_delta", 0):
            f.rope_delta = seq.rope_delta
        return f

    def release(self, seq):
        seq.release()


class _OracleSeq:
    def __init__(self, cache: ContiguousKvCache):
        self.cache = cache


class OracleBackend:
    def __init__(self, model: OracleLlama, max_context: int = 8192):
        self.model = model
        self.vocab_size = model.cfg.vocab_size
        self.max_context = max_context

    def new_sequence(self) -> _OracleSeq:
        return _OracleSeq(self.model.make_cache())

    def length(self, seq):
        return seq.cache.offset

    def forward(self, seqs, new_tokens, all_positions=False):
        out = []
        ov = _take_overrides(seqs) or [None] * len(seqs)
        for s, toks, o in zip(seqs, new_tokens, ov):
            ids = torch.tensor([toks], dtype=torch.long)
            kw = {}
            if o is not None:
                emb = self.model.embed(ids.to(self.model.device)).clone()
                emb[0, o[0]] = o[1].to(emb.device, emb.dtype)
                kw["embeds"] = emb
            mr = getattr(s, "pending_mrope", None)
            offset = s.cache.offset + getattr(s, "rope_delta", 0)
            if mr is not None:
                s.pending_mrope = None
                kw["mrope_positions"], kw["deepstack"] = mr[0], (mr[2], mr[3])
                s.rope_delta = mr[1] - (s.cache.offset + len(toks))
            if all_positions:
                out.append(self.model.decode_logits_all(ids, s.cache, offset, **kw)[0].float())
            else:
                out.append(self.model.decode_logits(ids, s.cache, offset, **kw)[0].float())
        return out

    def forward_greedy(self, seqs, new_tokens):
        return [int(torch.argmax(l)) for l in self.forward(seqs, new_tokens)]

    def truncate(self, seq, length):
        seq.cache.truncate(length)

    def fork(self, seq, n_tokens):
        c = seq.cache.clone()
        c.truncate(n_tokens)
        f = _OracleSeq(c)
        if getattr(seq, "rope_delta", 0):
            f.rope_delta = seq.rope_delta
        return f

    def release(self, seq):
        seq.cache.reset()
