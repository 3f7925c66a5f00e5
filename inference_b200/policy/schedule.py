"""Iteration-level batching bookkeeping: budgets, stop tokens, finish reasons (core-llm/src/schedule.rs:49-223).
A stop token is excluded from the output, the budget-filling token is included, a zero-budget request is
admitted already finished."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

from ..contracts.core_llm.output import FinishReason
from ._lib import i32_array, lib

_REASON = {0: None, 1: FinishReason.STOP, 2: FinishReason.LENGTH}


@dataclass
class SeqSpec:
    prompt_tokens: list[int]
    max_new_tokens: int
    stop_tokens: list[int] = field(default_factory=list)


class Scheduler:
    def __init__(self):
        self._lib = lib()
        self._h = self._lib.swb_sched_new()

    def __del__(self):
        try:
            self._lib.swb_sched_free(self._h)
        except Exception:
            pass

    def admit(self, spec: SeqSpec) -> int:
        return self._lib.swb_sched_admit(self._h, len(spec.prompt_tokens), spec.max_new_tokens,
                                         i32_array(spec.stop_tokens), len(spec.stop_tokens))

    def __len__(self) -> int:
        return self._lib.swb_sched_len(self._h)

    def _list(self, finished: bool) -> list[int]:
        n = len(self)
        buf = (ctypes.c_long * max(1, n))()
        k = self._lib.swb_sched_list(self._h, 1 if finished else 0, buf, n)
        return list(buf[:k])

    def active(self) -> list[int]:
        return self._list(False)

    def finished(self) -> list[int]:
        return self._list(True)

    def is_active(self, seq: int) -> bool:
        return 0 <= seq < len(self) and self._lib.swb_sched_finish_reason(self._h, seq) == 0

    def all_finished(self) -> bool:
        return not self.active()

    def record(self, seq: int, token: int) -> FinishReason | None:
        r = self._lib.swb_sched_record(self._h, seq, token)
        return _REASON.get(r) if r > 0 else None

    def generated(self, seq: int) -> list[int]:
        n = self._lib.swb_sched_generated(self._h, seq, None, 0)
        buf = (ctypes.c_int32 * max(1, n))()
        self._lib.swb_sched_generated(self._h, seq, buf, n)
        return list(buf[:n])

    def finish_reason(self, seq: int) -> FinishReason | None:
        return _REASON[self._lib.swb_sched_finish_reason(self._h, seq)]

    def prompt_len(self, seq: int) -> int:
        return self._lib.swb_sched_prompt_len(self._h, seq)

    def offset(self, seq: int) -> int:
        return self._lib.swb_sched_offset(self._h, seq)
