"""Generation loops over a DecodeBackend: streaming single-sequence decode, synchronous batching, iteration-level
continuous batching, prefix-cached generation and speculative decoding (prompt lookup and draft model).

Behavioural parity: candle-llm/src/decode/stream.rs:65-305 (generate / decode_loop), batch.rs:54-283,
continuous.rs:45-491, prefix.rs:39-230, speculative.rs:46-464. Laws kept: batched == solo, continuous(Exact) ==
solo, prefix-cached == cold, greedy speculative == plain greedy token for token."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..contracts.core_llm.cancel import CancelFlag
from ..contracts.core_llm.output import FinishReason
from ..policy import sampler as hs
from ..policy.prefix import PrefixIndex
from ..policy.schedule import Scheduler, SeqSpec
from ..policy.speculative import accept_greedy_run, accept_token, ngram_propose, sample_weighted
from .backend import DecodeBackend


@dataclass
class GenerationConfig:
    max_new_tokens: int = 128
    sampling: hs.SamplingParams = field(default_factory=hs.SamplingParams)
    seed: int = 0
    stop_tokens: tuple[int, ...] = ()
    cancel: CancelFlag | None = None
    device_sampling: bool | None = None      # None: on the device when several rows step together, else on the host


@dataclass
class GenerationResult:
    tokens: list[int]
    finish_reason: FinishReason
    prompt_tokens: int = 0


AllowMask = Callable[[list[int]], "list[bool] | None"]   # generated-so-far -> allow mask (or None)
TokenSink = Callable[[int], bool]                         # return False to stop


def _pick(backend: DecodeBackend, logits: torch.Tensor, history: list[int], cfg: GenerationConfig, rng: hs.SplitMix64,
          allowed) -> int:
    if cfg.sampling.is_plain_greedy() and allowed is None:
        return int(torch.argmax(logits))
    return hs.sample(logits.detach().float().cpu().numpy(), history, cfg.sampling, rng, allowed)


def decode_loop(backend: DecodeBackend, seq: Any, first_logits: torch.Tensor | None, first_token: int | None,
                cfg: GenerationConfig, sink: TokenSink | None = None, mask: AllowMask | None = None,
                prompt: list[int] | None = None) -> tuple[list[int], FinishReason]:
    """Shared token loop: sample, check stop / sink / budget, step. `first_logits` (or a pre-sampled greedy
    `first_token`) come from the prefill. The repetition-penalty window is the prompt followed by the generated
    tokens (candle-llm/src/decode/stream.rs:210-285 seeds the history with the prompt ids); the allow mask sees the
    generated tokens only."""
    rng = hs.SplitMix64(cfg.seed)
    out: list[int] = []
    history: list[int] = list(prompt) if prompt is not None else []
    logits, tok = first_logits, first_token
    greedy_fast = cfg.sampling.is_plain_greedy() and mask is None
    for _ in range(cfg.max_new_tokens):
        if cfg.cancel is not None and cfg.cancel.is_cancelled():
            return out, FinishReason.CANCELLED
        if tok is None:
            tok = _pick(backend, logits, history, cfg, rng, mask(out) if mask else None)
        if tok in cfg.stop_tokens:
            return out, FinishReason.STOP
        out.append(tok)
        history.append(tok)
        if sink is not None and sink(tok) is False:
            return out, FinishReason.STOP
        if len(out) >= cfg.max_new_tokens:
            return out, FinishReason.LENGTH
        if greedy_fast:
            tok = backend.forward_greedy([seq], [[tok]])[0]
        else:
            logits = backend.forward([seq], [[tok]])[0]
            tok = None
    return out, FinishReason.LENGTH


def generate(backend: DecodeBackend, prompt: list[int], cfg: GenerationConfig, sink: TokenSink | None = None,
             mask: AllowMask | None = None, seq: Any | None = None) -> GenerationResult:
    """Prefill (whatever of `prompt` the sequence does not hold yet) then the token loop."""
    own = seq is None
    seq = backend.new_sequence() if own else seq
    try:
        have = backend.length(seq)
        suffix = prompt[have:]
        if cfg.max_new_tokens <= 0:
            return GenerationResult([], FinishReason.LENGTH, len(prompt))
        if cfg.cancel is not None and cfg.cancel.is_cancelled():
            return GenerationResult([], FinishReason.CANCELLED, len(prompt))
        if cfg.sampling.is_plain_greedy() and mask is None:
            first = backend.forward_greedy([seq], [suffix])[0]
            toks, why = decode_loop(backend, seq, None, first, cfg, sink, mask, prompt=prompt)
        else:
            logits = backend.forward([seq], [suffix])[0]
            toks, why = decode_loop(backend, seq, logits, None, cfg, sink, mask, prompt=prompt)
        return GenerationResult(toks, why, len(prompt))
    finally:
        if own:
            backend.release(seq)


def _device_sampling(cfg: GenerationConfig, logits: torch.Tensor, rows: int) -> bool:
    """Stochastic rows are drawn on the device when the logits live there, no repetition penalty reshapes them and
    either the request asked for it or more than one row steps together (the host sampler reproduces the reference's
    token stream for a seed; the device sampler draws from the same distribution with its own index order, so single
    sequences stay on the host path unless `device_sampling` is set)."""
    sp = cfg.sampling
    if not isinstance(logits, torch.Tensor) or not logits.is_cuda or sp.temperature <= 0.0 or sp.repetition_penalty != 1.0:
        return False
    want = getattr(cfg, "device_sampling", None)
    return bool(want) if want is not None else rows > 1


def ops_sample_device(logits, temperature, top_k, top_p, uniforms):
    from .. import ops

    l2 = logits if logits.dtype in (torch.float32, torch.bfloat16) else logits.float()
    return ops.sample_device(l2.contiguous(), temperature, top_k, top_p, uniforms)


def generate_batch(backend: DecodeBackend, prompts: list[list[int]], cfg: GenerationConfig) -> list[GenerationResult]:
    """Synchronous batched greedy/stochastic decode: one ragged prefill, then lock-step steps over the live rows
    (rows retire independently; no padding, no masks)."""
    seqs = [backend.new_sequence() for _ in prompts]
    rngs = [hs.SplitMix64(cfg.seed + i) for i in range(len(prompts))]
    sched = Scheduler()
    ids = [sched.admit(SeqSpec(p, cfg.max_new_tokens, list(cfg.stop_tokens))) for p in prompts]
    try:
        greedy = cfg.sampling.is_plain_greedy()
        live = [i for i in ids if sched.is_active(i)]
        new = [prompts[i] for i in live]
        while live:
            if cfg.cancel is not None and cfg.cancel.is_cancelled():
                break
            if greedy:
                toks = backend.forward_greedy([seqs[i] for i in live], new)
            else:
                logits = backend.forward([seqs[i] for i in live], new)
                if _device_sampling(cfg, logits, len(live)):
                    # one kernel for all rows; each row consumes one number of its own stream per step
                    u = torch.tensor([rngs[i].next_f32() for i in live], dtype=torch.float32).to(logits.device, non_blocking=True)
                    sp = cfg.sampling
                    toks = [int(t) for t in ops_sample_device(logits, sp.temperature, sp.top_k, sp.top_p, u).tolist()]
                else:
                    # penalty window = prompt + generated (candle-llm/src/decode/batch.rs:133)
                    toks = [_pick(backend, logits[k], list(prompts[i]) + sched.generated(i), cfg, rngs[i], None)
                            for k, i in enumerate(live)]
            nxt, new = [], []
            for k, i in enumerate(live):
                if sched.record(i, toks[k]) is None:
                    nxt.append(i)
                    new.append([toks[k]])
            live = nxt
        res = []
        for i in ids:
            why = sched.finish_reason(i) or FinishReason.CANCELLED
            res.append(GenerationResult(sched.generated(i), why, len(prompts[i])))
        return res
    finally:
        for s in seqs:
            backend.release(s)


class BatchExactness(enum.Enum):
    EXACT = "exact"            # every sequence steps alone: bit-identical to a solo run
    THROUGHPUT = "throughput"  # live sequences step together in one batched forward


@dataclass
class ContinuousConfig:
    max_batch: int = 8
    block_size: int = 16
    exactness: BatchExactness = BatchExactness.THROUGHPUT
    prefill_chunk: int = 0        # > 0: at most this many prompt tokens per step, in the same forward as the decode rows


@dataclass
class ContinuousRequest:
    prompt: list[int]
    max_new_tokens: int
    stop_tokens: tuple[int, ...] = ()


def generate_continuous(backend: DecodeBackend, requests: list[ContinuousRequest], ccfg: ContinuousConfig,
                        sink: Callable[[int, int], None] | None = None, cancel: CancelFlag | None = None
                        ) -> list[GenerationResult]:
    """Iteration-level (continuous) batching with admit-on-retire: at most max_batch sequences are live; when one
    retires its KV blocks are released and the next pending request is prefilled into the freed slot."""
    sched = Scheduler()
    ids = [sched.admit(SeqSpec(r.prompt, r.max_new_tokens, list(r.stop_tokens))) for r in requests]
    pending = [i for i in ids if sched.is_active(i)]
    lanes: dict[int, Any] = {}
    next_tok: dict[int, int] = {}
    fed: dict[int, int] = {}          # chunked prefill: prompt tokens already fed per lane still in its prompt
    exact = ccfg.exactness is BatchExactness.EXACT

    def step(group: list[int], new: list[list[int]], unfinished: frozenset | set = frozenset()) -> None:
        if exact:
            toks = [backend.forward_greedy([lanes[i]], [n])[0] for i, n in zip(group, new)]
        else:
            toks = backend.forward_greedy([lanes[i] for i in group], new)
        for i, t in zip(group, toks):
            if i in unfinished:          # a prompt chunk that does not end the prompt: its logits predict nothing yet
                continue
            why = sched.record(i, t)
            if why is None or why is FinishReason.LENGTH:
                if sink is not None:
                    sink(i, t)
            if why is None:
                next_tok[i] = t
            else:
                backend.release(lanes.pop(i))
                next_tok.pop(i, None)

    try:
        while pending or lanes:
            if cancel is not None and cancel.is_cancelled():
                break
            # admit into free slots: the admitted prompts prefill together in one ragged forward
            admitted = []
            while pending and len(lanes) < ccfg.max_batch:
                i = pending.pop(0)
                lanes[i] = backend.new_sequence()
                admitted.append(i)
            if ccfg.prefill_chunk > 0:
                # chunked prefill: decode rows and a bounded slice of prompt tokens share one ragged forward, so a long
                # prompt never stalls the running sequences for more than one chunk
                for i in admitted:
                    fed[i] = 0
                group = [i for i in lanes if i in next_tok]
                new = [[next_tok[i]] for i in group]
                budget, unfinished = ccfg.prefill_chunk, set()
                for i in [j for j in lanes if j in fed]:
                    if budget <= 0:
                        break
                    prompt, s0 = requests[i].prompt, fed[i]
                    n = min(budget, len(prompt) - s0)
                    group.append(i)
                    new.append(prompt[s0:s0 + n])
                    budget -= n
                    if s0 + n < len(prompt):
                        fed[i] = s0 + n
                        unfinished.add(i)
                    else:
                        del fed[i]
                if group:
                    step(group, new, unfinished)
                continue
            if admitted:
                step(admitted, [requests[i].prompt for i in admitted])
            live = [i for i in lanes if i in next_tok and i not in admitted]
            if live:
                step(live, [[next_tok[i]] for i in live])
        return [GenerationResult(sched.generated(i), sched.finish_reason(i) or FinishReason.CANCELLED,
                                 len(requests[i].prompt)) for i in ids]
    finally:
        for s in lanes.values():
            backend.release(s)


# ---- prefix cache -------------------------------------------------------------------------------------------
@dataclass
class PrefixStats:
    lookups: int = 0
    hits: int = 0
    reused_tokens: int = 0
    computed_tokens: int = 0


class PrefixCache:
    """LRU cache of prompt KV state keyed by token prefix. A hit seeds a new sequence with the shared prefix
    (copy-on-write on paged backends), the rest of the prompt is prefilled, and the finished prompt is stored."""

    def __init__(self, backend: DecodeBackend, capacity: int = 8):
        self.backend = backend
        self.index = PrefixIndex(capacity)
        self.entries: dict[int, tuple[Any, int]] = {}   # PrefixId -> (sequence holding the prompt KV, length)
        self.stats = PrefixStats()

    def seed(self, prompt: list[int]) -> Any:
        """A sequence pre-populated with the longest cached prefix of `prompt` (always leaves >= 1 token to run)."""
        self.stats.lookups += 1
        m = self.index.longest_match(prompt)
        if m is not None and m.id in self.entries:
            src, length = self.entries[m.id]
            n = min(m.matched_len, length, len(prompt) - 1)
            if n > 0:
                seq = self.backend.fork(src, n)
                reused = self.backend.length(seq)
                if reused > 0:
                    self.stats.hits += 1
                    self.stats.reused_tokens += reused
                    return seq
                self.backend.release(seq)
        return self.backend.new_sequence()

    def store(self, prompt: list[int], seq: Any) -> None:
        """Keeps a snapshot of `seq` truncated to the prompt (generated tokens are not part of the key)."""
        snap = self.backend.fork(seq, len(prompt))
        out = self.index.insert(list(prompt))
        old = self.entries.pop(out.id, None)
        if old is not None:
            self.backend.release(old[0])
        self.entries[out.id] = (snap, self.backend.length(snap))
        for ev in out.evicted:
            e = self.entries.pop(ev, None)
            if e is not None:
                self.backend.release(e[0])

    def clear(self) -> None:
        for s, _ in self.entries.values():
            self.backend.release(s)
        self.entries.clear()


def generate_cached(backend: DecodeBackend, cache: PrefixCache, prompt: list[int], cfg: GenerationConfig,
                    sink: TokenSink | None = None) -> GenerationResult:
    seq = cache.seed(prompt)
    try:
        cache.stats.computed_tokens += len(prompt) - backend.length(seq)
        if cfg.sampling.is_plain_greedy():
            first = backend.forward_greedy([seq], [prompt[backend.length(seq):]])[0]
            cache.store(prompt, seq)
            toks, why = decode_loop(backend, seq, None, first, cfg, sink, prompt=prompt)
        else:
            logits = backend.forward([seq], [prompt[backend.length(seq):]])[0]
            cache.store(prompt, seq)
            toks, why = decode_loop(backend, seq, logits, None, cfg, sink, prompt=prompt)
        return GenerationResult(toks, why, len(prompt))
    finally:
        backend.release(seq)


# ---- speculative decoding -------------------------------------------------------------------------------------
@dataclass
class SpeculativeConfig:
    max_ngram: int = 3
    num_draft: int = 4


@dataclass
class SpeculativeStats:
    forwards: int = 0     # target forwards (prefill included)
    proposed: int = 0
    accepted: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0


def _verify(target: DecodeBackend, seq: Any, last: int, drafts: list[int], draft_dists, cfg: GenerationConfig,
            rng: hs.SplitMix64, history: list[int]) -> tuple[list[int], int]:
    """One target forward over [last, d_1..d_k]; returns (tokens to emit, number of drafts accepted). `history` is
    the penalty window up to and including `last` (prompt + emitted tokens), the same list the draft shapes q with."""
    base = target.length(seq)
    logits = target.forward([seq], [[last] + drafts], all_positions=True)[0]   # [k + 1, vocab]
    if cfg.sampling.temperature <= 0.0:
        if cfg.sampling.is_plain_greedy():
            argmax = [int(x) for x in torch.argmax(logits, dim=-1).tolist()]
        else:
            # penalty-aware argmax per verify position, the window growing by the drafts
            # (candle-llm/src/decode/speculative.rs:399-421)
            argmax, hist = [], list(history)
            rows = logits.detach().float().cpu().numpy()
            for i in range(len(drafts) + 1):
                argmax.append(hs.sample(rows[i], hist, cfg.sampling, rng, None))
                if i < len(drafts):
                    hist.append(drafts[i])
        n = accept_greedy_run(argmax, drafts)
        emit = drafts[:n] + [argmax[n]]
    else:
        emit, n = [], 0
        hist = list(history)
        for i, d in enumerate(drafts):
            p = hs.shaped_candidates(logits[i].float().cpu().numpy(), hist, cfg.sampling)
            ok, tok = accept_token(p, draft_dists[i], d, rng.next_f32(), rng.next_f32())
            emit.append(tok)
            hist.append(tok)
            if not ok:
                break
            n += 1
        else:
            p = hs.shaped_candidates(logits[len(drafts)].float().cpu().numpy(), hist, cfg.sampling)
            emit.append(sample_weighted(p, rng.next_f32(), p[0][0] if p else 0))
    # keep KV for `last` and the accepted drafts only; the emitted bonus / correction token is fed next round
    target.truncate(seq, base + 1 + n)
    return emit, n


def _spec_loop(target: DecodeBackend, prompt: list[int], cfg: GenerationConfig, propose, on_accept, sink
               ) -> tuple[GenerationResult, SpeculativeStats]:
    stats = SpeculativeStats()
    rng = hs.SplitMix64(cfg.seed)
    seq = target.new_sequence()
    out: list[int] = []
    why = FinishReason.LENGTH
    try:
        if cfg.max_new_tokens <= 0:
            return GenerationResult([], FinishReason.LENGTH, len(prompt)), stats
        logits = target.forward([seq], [prompt])[0]
        stats.forwards += 1
        last = _pick(target, logits, list(prompt), cfg, rng, None)
        done = False
        while not done:
            if cfg.cancel is not None and cfg.cancel.is_cancelled():
                why = FinishReason.CANCELLED
                break
            if last in cfg.stop_tokens:
                why = FinishReason.STOP
                break
            out.append(last)
            if sink is not None and sink(last) is False:
                why = FinishReason.STOP
                break
            if len(out) >= cfg.max_new_tokens:
                break
            budget = cfg.max_new_tokens - len(out)
            drafts, dists = propose(prompt + out, min(budget - 1, 1 << 30))
            emit, n = _verify(target, seq, last, drafts, dists, cfg, rng, prompt + out)
            stats.forwards += 1
            stats.proposed += len(drafts)
            stats.accepted += n
            on_accept(len(prompt) + len(out) + n)
            # all but the final emitted token are accepted drafts: stream them, the final one loops as `last`
            for t in emit[:-1]:
                if t in cfg.stop_tokens:
                    why, done = FinishReason.STOP, True
                    break
                out.append(t)
                if sink is not None and sink(t) is False:
                    why, done = FinishReason.STOP, True
                    break
                if len(out) >= cfg.max_new_tokens:
                    done = True
                    break
            last = emit[-1]
        return GenerationResult(out, why, len(prompt)), stats
    finally:
        target.release(seq)


def generate_prompt_lookup(target: DecodeBackend, prompt: list[int], cfg: GenerationConfig,
                           spec: SpeculativeConfig | None = None, sink: TokenSink | None = None
                           ) -> tuple[GenerationResult, SpeculativeStats]:
    """Speculative decoding without a draft model: proposals are continuations of the most recent matching n-gram."""
    spec = spec or SpeculativeConfig()

    def propose(tokens, room):
        d = ngram_propose(tokens, spec.max_ngram, max(0, min(spec.num_draft, room)))
        return d, [[(t, 1.0)] for t in d]   # point-mass proposal distributions

    return _spec_loop(target, prompt, cfg, propose, lambda _n: None, sink)


def generate_draft_speculative(target: DecodeBackend, draft: DecodeBackend, prompt: list[int], cfg: GenerationConfig,
                               spec: SpeculativeConfig | None = None, sink: TokenSink | None = None
                               ) -> tuple[GenerationResult, SpeculativeStats]:
    """Draft-model speculative decoding: the draft proposes num_draft tokens autoregressively (recording its
    shaped distribution q_i), the target scores all of them in one forward, acceptance preserves the target
    distribution; both caches roll back to the accepted length."""
    spec = spec or SpeculativeConfig()
    dseq = draft.new_sequence()
    drng = hs.SplitMix64(cfg.seed ^ 0x5DEECE66D)
    state = {"fed": 0}

    def propose(tokens, room):
        k = max(0, min(spec.num_draft, room))
        if k == 0:
            return [], []
        feed = tokens[state["fed"]:]
        drafts, dists = [], []
        hist = list(tokens)
        for _ in range(k):
            logits = draft.forward([dseq], [feed])[0]
            state["fed"] += len(feed)
            if cfg.sampling.temperature <= 0.0:
                t = int(torch.argmax(logits))
                q = [(t, 1.0)]
            else:
                q = hs.shaped_candidates(logits.float().cpu().numpy(), hist, cfg.sampling)
                t = sample_weighted(q, drng.next_f32(), q[0][0] if q else 0)
            drafts.append(t)
            dists.append(q)
            hist.append(t)
            feed = [t]
        return drafts, dists

    def on_accept(valid_len):
        # the draft cache holds tokens[:fed]; keep only what the target accepted
        keep = min(state["fed"], valid_len)
        draft.truncate(dseq, keep)
        state["fed"] = keep

    try:
        return _spec_loop(target, prompt, cfg, propose, on_accept, sink)
    finally:
        draft.release(dseq)
