"""Component residency for two-phase media pipelines (parity: candle-gen/src/residency.rs:160-330).

A pipeline has a light phase (text encoders) and a heavy phase (transformer + VAE). `Resident` keeps both cached
after first use; `Sequential` loads the text encoders, encodes, synchronises the device, drops them, and only then
loads the heavy phase, so peak memory is max(phase) instead of the sum. With 180 GB per GPU the resident policy is
the default; sequential remains for very large text encoders or many co-resident models."""
from __future__ import annotations

import threading
from typing import Any, Callable

from ..contracts.errors import Canceled
from ..contracts.gen_core.runtime import CancelFlag, LoadPhase, OffloadPolicy, ProgressLoading


class Residency:
    def __init__(self, policy: OffloadPolicy, load_text: Callable[[], Any], load_heavy: Callable[[], Any],
                 synchronize: Callable[[], None] = lambda: None):
        self.policy = policy
        self._load_text, self._load_heavy, self._sync = load_text, load_heavy, synchronize
        self._lock = threading.Lock()
        self._text = None
        self._heavy = None

    @staticmethod
    def from_policy(policy: OffloadPolicy | None, load_text, load_heavy, synchronize=lambda: None) -> "Residency":
        return Residency(policy or OffloadPolicy.RESIDENT, load_text, load_heavy, synchronize)

    def loaded_phases(self) -> tuple[bool, bool]:
        return self._text is not None, self._heavy is not None

    def run(self, cancel: CancelFlag, on_progress, encode: Callable[[Any], Any], render: Callable[[Any, Any], Any]):
        """encode(text_components) -> conditioning; render(heavy_components, conditioning) -> result."""
        def check():
            if cancel.is_cancelled():
                raise Canceled("generation cancelled")

        with self._lock:      # one generation at a time per loaded model, like the reference's component mutex
            check()
            if self.policy is OffloadPolicy.RESIDENT:
                if self._text is None:
                    on_progress(ProgressLoading(LoadPhase.TEXT_ENCODER))
                    self._text = self._load_text()
                check()
                cond = encode(self._text)
                check()
                if self._heavy is None:
                    on_progress(ProgressLoading(LoadPhase.TRANSFORMER))
                    self._heavy = self._load_heavy()
                check()
                return render(self._heavy, cond)
            on_progress(ProgressLoading(LoadPhase.TEXT_ENCODER))
            text = self._load_text()
            try:
                check()
                cond = encode(text)
                self._sync()          # the encoders' work must be finished before their memory goes back
            finally:
                del text
            check()
            on_progress(ProgressLoading(LoadPhase.TRANSFORMER))
            heavy = self._load_heavy()
            try:
                check()
                out = render(heavy, cond)
                self._sync()
                return out
            finally:
                del heavy
