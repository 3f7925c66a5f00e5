"""Process-local counters, gauges and latency histograms with a Prometheus text rendering (no dependency on a
client library). The reference has no metrics endpoint (its observability is `tracing` spans and bench harness
reports); this is what the serving front end exposes at GET /metrics."""
from __future__ import annotations

import bisect
import threading

_BUCKETS = (0.001, 0.0025, 0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0)


class Metrics:
    def __init__(self, prefix: str = "swb"):
        self.prefix = prefix
        self._lock = threading.Lock()
        self._counters: dict[str, float] = {}
        self._gauges: dict[str, float] = {}
        self._hist: dict[str, tuple[list[int], float, int]] = {}

    def inc(self, name: str, by: float = 1.0) -> None:
        with self._lock:
            self._counters[name] = self._counters.get(name, 0.0) + by

    def set(self, name: str, value: float) -> None:
        with self._lock:
            self._gauges[name] = float(value)

    def add_gauge(self, name: str, by: float) -> None:
        with self._lock:
            self._gauges[name] = self._gauges.get(name, 0.0) + by

    def observe(self, name: str, seconds: float) -> None:
        with self._lock:
            counts, total, n = self._hist.get(name, ([0] * (len(_BUCKETS) + 1), 0.0, 0))
            counts[bisect.bisect_left(_BUCKETS, seconds)] += 1
            self._hist[name] = (counts, total + seconds, n + 1)

    def snapshot(self) -> dict:
        with self._lock:
            return {"counters": dict(self._counters), "gauges": dict(self._gauges),
                    "histograms": {k: {"count": v[2], "sum": v[1]} for k, v in self._hist.items()}}

    def quantile(self, name: str, q: float) -> float | None:
        """Upper bucket bound below which a fraction q of the observations fall."""
        with self._lock:
            if name not in self._hist or self._hist[name][2] == 0:
                return None
            counts, _, n = self._hist[name]
        acc = 0
        for i, c in enumerate(counts):
            acc += c
            if acc >= q * n:
                return _BUCKETS[i] if i < len(_BUCKETS) else float("inf")
        return float("inf")

    def render_prometheus(self) -> str:
        out = []
        with self._lock:
            for k, v in sorted(self._counters.items()):
                out += [f"# TYPE {self.prefix}_{k} counter", f"{self.prefix}_{k} {v:g}"]
            for k, v in sorted(self._gauges.items()):
                out += [f"# TYPE {self.prefix}_{k} gauge", f"{self.prefix}_{k} {v:g}"]
            for k, (counts, total, n) in sorted(self._hist.items()):
                out.append(f"# TYPE {self.prefix}_{k} histogram")
                acc = 0
                for b, c in zip(_BUCKETS, counts):
                    acc += c
                    out.append(f'{self.prefix}_{k}_bucket{{le="{b:g}"}} {acc}')
                out.append(f'{self.prefix}_{k}_bucket{{le="+Inf"}} {n}')
                out += [f"{self.prefix}_{k}_sum {total:g}", f"{self.prefix}_{k}_count {n}"]
        return "\n".join(out) + "\n"


GLOBAL = Metrics()
