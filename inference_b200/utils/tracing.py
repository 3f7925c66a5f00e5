"""Span timing for host code and CUDA-event timing for device work; spans nest per thread and are exported as a
Chrome-trace JSON (the reference's tracing story is `tracing` spans plus per-stage timers in its bench harnesses)."""
from __future__ import annotations

import json
import threading
import time
from contextlib import contextmanager

_local = threading.local()
_events: list[dict] = []
_lock = threading.Lock()
enabled = False


def enable(on: bool = True) -> None:
    global enabled
    enabled = on


nvtx_enabled = False


def enable_nvtx(on: bool = True) -> None:
    """Also open an NVTX range per span (visible to profilers that show NVTX; costs two driver calls per span)."""
    global nvtx_enabled
    nvtx_enabled = on


@contextmanager
def span(name: str, **args):
    if not enabled and not nvtx_enabled:
        yield
        return
    pushed = False
    if nvtx_enabled:
        try:
            import torch

            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:  # noqa: BLE001  (no CUDA runtime: host spans only)
            pushed = False
    t0 = time.perf_counter_ns()
    try:
        yield
    finally:
        t1 = time.perf_counter_ns()
        if pushed:
            import torch

            torch.cuda.nvtx.range_pop()
        if not enabled:
            return
        with _lock:
            _events.append({"name": name, "ph": "X", "ts": t0 / 1e3, "dur": (t1 - t0) / 1e3, "pid": 0,
                            "tid": threading.get_ident() % 100000, "args": args})


class DeviceTimer:
    """CUDA-event stopwatch on the current stream: `with DeviceTimer() as t: ...; t.ms` (synchronises on exit)."""

    def __enter__(self):
        import torch

        self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._e0.record()
        return self

    def __exit__(self, *exc):
        import torch

        self._e1.record()
        torch.cuda.synchronize()
        self.ms = self._e0.elapsed_time(self._e1)


def export_chrome_trace(path: str) -> int:
    with _lock:
        ev = list(_events)
    with open(path, "w") as f:
        json.dump({"traceEvents": ev}, f)
    return len(ev)


def clear() -> None:
    with _lock:
        _events.clear()


# ---- device launch timeline ---------------------------------------------------------------------------------
TIMELINE_IDS = {0: "other", 1: "embedding", 2: "rmsnorm", 3: "gemm_decode_cluster", 4: "rope_kv_write", 5: "attn_decode",
                6: "attn_merge", 7: "gemm_tcgen05", 8: "argmax", 9: "argmax_merge", 10: "decode_meta_unpack",
                11: "decode_step_tail", 12: "peer_collective", 13: "gated_act_mul", 14: "attn_prefill", 15: "gemm_quant"}


class LaunchTimeline:
    """Per-launch device timestamps of this library's kernels, CUDA graphs included (each kernel's block 0 stamps the
    global timer before and after its programmatic-dependency wait). `with LaunchTimeline() as tl: <launch work>` then
    `tl.records()`: one dict per launch in start order with `name`, `grid`, `entered_ns` (block 0 reached its wait),
    `released_ns` (its predecessor had completely finished) and `span_ns` (released -> the next launch's release, i.e.
    this launch's contribution to the critical path). Times are relative to the first record."""

    def __init__(self, capacity: int = 4096):
        self.capacity = capacity
        self._buf = None

    def __enter__(self):
        import torch

        from .._native import kernels

        self._buf = torch.zeros(8 + 4 * self.capacity, dtype=torch.int64, device="cuda")
        self._buf[1] = self.capacity
        torch.cuda.synchronize()
        kernels().swb_set_timeline(self._buf.data_ptr())
        return self

    def __exit__(self, *exc):
        import torch

        from .._native import kernels

        torch.cuda.synchronize()
        kernels().swb_set_timeline(None)
        self._host = self._buf.cpu()
        self._buf = None

    def records(self) -> list[dict]:
        h = self._host
        n = min(int(h[0]), self.capacity)
        rec = h[8:8 + 4 * n].view(n, 4).tolist()
        rec.sort(key=lambda r: r[2])
        if not rec:
            return []
        t0 = rec[0][1]
        out = []
        for i, (kid, a, b, grid) in enumerate(rec):
            nxt = rec[i + 1][2] if i + 1 < n else None
            out.append({"name": TIMELINE_IDS.get(kid, str(kid)), "grid": grid, "entered_ns": a - t0,
                        "released_ns": b - t0, "span_ns": (nxt - b) if nxt is not None else None})
        return out

    @staticmethod
    def summarize(records: list[dict]) -> list[dict]:
        """Totals per (kernel, grid): launches, critical-path share (sum of span_ns) and mean head start (how long
        block 0 sat in its wait: the part of the launch that overlapped its predecessor)."""
        agg: dict[tuple[str, int], list[float]] = {}
        for r in records:
            a = agg.setdefault((r["name"], r["grid"]), [0, 0.0, 0.0])
            a[0] += 1
            a[1] += r["span_ns"] or 0
            a[2] += r["released_ns"] - r["entered_ns"]
        rows = [{"name": k[0], "grid": k[1], "launches": v[0], "span_us": round(v[1] / 1e3, 1),
                 "mean_span_us": round(v[1] / v[0] / 1e3, 2), "mean_head_start_us": round(v[2] / v[0] / 1e3, 2)}
                for k, v in agg.items()]
        rows.sort(key=lambda r: -r["span_us"])
        return rows
