"""Cross-request iteration-level batching as a `DecodeBackend` proxy.

Every client thread runs the ordinary single-request generation loop (sampling, constraints, stop handling stay per
request) against a `BatchingBackend`. Its forward calls do not run the model: they queue, and one worker thread
merges the calls that are waiting - decode steps of many requests into one batched decode, new prompts into one
ragged prefill - runs them on the real backend and hands each caller its slice. Sequence bookkeeping (new / fork /
truncate / release) is serialised with the worker so the paged allocator never changes under a running step.
The reference server handles one connection at a time and never batches across them
(candle-llm's scheduler is a library call: candle-llm/src/decode/continuous.rs); this is the serving-side use of it."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any


@dataclass
class _Call:
    kind: str                      # "greedy" | "logits"
    seqs: list[Any]
    new_tokens: list[list[int]]
    all_positions: bool = False
    done: threading.Event = field(default_factory=threading.Event)
    result: Any = None
    error: BaseException | None = None


@dataclass
class BatchingStats:
    steps: int = 0
    merged_calls: int = 0
    max_merged: int = 0
    rows: int = 0


class BatchingBackend:
    def __init__(self, inner, max_batch: int = 64, window_s: float = 0.002):
        self.inner, self.max_batch, self.window_s = inner, max_batch, window_s
        self.max_context = getattr(inner, "max_context", 0)
        self.stats = BatchingStats()
        self._lock = threading.Lock()            # guards the inner backend
        self._cv = threading.Condition()
        self._pending: list[_Call] = []
        self._clients = 0
        self._stop = False
        self._worker = threading.Thread(target=self._run, name="swb-batcher", daemon=True)
        self._worker.start()

    # ---- client registration: lets the worker skip the window when every client is already waiting -----------
    def __enter__(self):
        with self._cv:
            self._clients += 1
        return self

    def __exit__(self, *exc):
        with self._cv:
            self._clients -= 1
            self._cv.notify_all()

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        self._worker.join(timeout=5)

    # ---- bookkeeping calls -----------------------------------------------------------------------------------
    def new_sequence(self):
        with self._lock:
            return self.inner.new_sequence()

    def length(self, seq):
        return self.inner.length(seq)

    def truncate(self, seq, length):
        with self._lock:
            return self.inner.truncate(seq, length)

    def fork(self, seq, n_tokens):
        with self._lock:
            return self.inner.fork(seq, n_tokens)

    def release(self, seq):
        with self._lock:
            return self.inner.release(seq)

    # ---- model calls -------------------------------------------------------------------------------------------
    def _submit(self, call: _Call):
        with self._cv:
            if self._stop:
                raise RuntimeError("batching backend is closed")
            self._pending.append(call)
            self._cv.notify_all()
        call.done.wait()
        if call.error is not None:
            raise call.error
        return call.result

    def forward_greedy(self, seqs, new_tokens):
        return self._submit(_Call("greedy", list(seqs), [list(t) for t in new_tokens]))

    def forward(self, seqs, new_tokens, all_positions=False):
        return self._submit(_Call("logits", list(seqs), [list(t) for t in new_tokens], all_positions))

    # ---- worker ------------------------------------------------------------------------------------------------
    def _take(self) -> list[_Call]:
        with self._cv:
            while not self._pending and not self._stop:
                self._cv.wait(0.05)
            if self._stop:
                return []
            deadline = time.monotonic() + self.window_s
            while (len(self._pending) < max(1, min(self._clients, self.max_batch)) and
                   (left := deadline - time.monotonic()) > 0):
                self._cv.wait(left)
            calls, self._pending = self._pending, []
            return calls

    def _run(self) -> None:
        while True:
            calls = self._take()
            if not calls:
                with self._cv:
                    if self._stop:
                        for c in self._pending:
                            c.error = RuntimeError("batching backend is closed")
                            c.done.set()
                        return
                continue
            groups: dict[tuple, list[_Call]] = {}
            for c in calls:
                decode = all(len(t) == 1 for t in c.new_tokens)
                key = (c.kind, decode, c.all_positions)
                groups.setdefault(key, []).append(c)
            for (kind, _decode, allpos), group in groups.items():
                for lo in range(0, len(group), self.max_batch):
                    self._execute(kind, allpos, group[lo:lo + self.max_batch])

    def _execute(self, kind: str, all_positions: bool, group: list[_Call]) -> None:
        seqs = [s for c in group for s in c.seqs]
        toks = [t for c in group for t in c.new_tokens]
        try:
            with self._lock:
                out = (self.inner.forward_greedy(seqs, toks) if kind == "greedy"
                       else self.inner.forward(seqs, toks, all_positions))
            i = 0
            for c in group:
                n = len(c.seqs)
                c.result = out[i:i + n]
                i += n
            self.stats.steps += 1
            self.stats.merged_calls += len(group)
            self.stats.max_merged = max(self.stats.max_merged, len(group))
            self.stats.rows += len(seqs)
        except BaseException as e:      # hand the failure to every caller of the merged step
            for c in group:
                c.error = e
        finally:
            for c in group:
                c.done.set()
