"""Opt-in step profiler: host phase timings and CUDA-event GPU timings, summarised as one JSON log line.

Same knobs as the reference's feeding profile (``runtime/profiling.py:13-203`` there):
``CUBIC_SERVE_FEEDING_PROFILE=1`` switches it on, ``CUBIC_SERVE_FEEDING_PROFILE_STEPS`` (default 100) sets the
window; every metric keeps at most 4096 samples and the summary reports count / sum / p50 / p95.  GPU timings
use pre-allocated CUDA events that are only read once complete, so profiling never adds a synchronisation.
NVTX ranges (``nvtx_range``) mark the same phases for external tools.
"""
from __future__ import annotations

import contextlib
import json
import logging
import os
import time
from collections import defaultdict

log = logging.getLogger("cubic.profile")
MAX_SAMPLES = 4096


def profiling_enabled() -> bool:
    return os.environ.get("CUBIC_SERVE_FEEDING_PROFILE", "0") not in ("", "0", "false")


class StepProfile:
    def __init__(self, window_steps: int | None = None, sink=None) -> None:
        self.window = window_steps or int(os.environ.get("CUBIC_SERVE_FEEDING_PROFILE_STEPS", "100"))
        self.samples: dict[str, list[float]] = defaultdict(list)
        self.steps = 0
        self.sink = sink or (lambda line: log.info("%s", line))

    def record(self, metric: str, ms: float) -> None:
        s = self.samples[metric]
        if len(s) < MAX_SAMPLES:
            s.append(float(ms))

    @contextlib.contextmanager
    def phase(self, metric: str):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.record(metric, (time.perf_counter() - t0) * 1e3)

    def end_step(self) -> dict | None:
        self.steps += 1
        if self.steps < self.window:
            return None
        summary = self.summary()
        self.sink(json.dumps({"feeding_profile": summary}))
        self.samples.clear()
        self.steps = 0
        return summary

    def summary(self) -> dict:
        out = {}
        for name, vals in self.samples.items():
            v = sorted(vals)
            n = len(v)
            out[name] = {"count": n, "sum_ms": round(sum(v), 3), "p50_ms": round(v[n // 2], 4),
                         "p95_ms": round(v[min(n - 1, int(n * 0.95))], 4)}
        return out


class CudaStepProfiler:
    """Ring of CUDA event pairs; a pair is harvested only when its end event has completed."""

    def __init__(self, profile: StepProfile, depth: int = 8) -> None:
        import torch
        self.profile = profile
        self.free = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(depth)]
        self.pending: list[tuple[str, object, object]] = []

    def begin(self, metric: str, stream):
        if not self.free:
            return None
        a, b = self.free.pop()
        a.record(stream)
        return (metric, a, b)

    def end(self, handle, stream) -> None:
        if handle is None:
            return
        handle[2].record(stream)
        self.pending.append(handle)
        self.harvest()

    def harvest(self) -> None:
        keep = []
        for metric, a, b in self.pending:
            if b.query():
                self.profile.record(metric, a.elapsed_time(b))
                self.free.append((a, b))
            else:
                keep.append((metric, a, b))
        self.pending = keep


@contextlib.contextmanager
def nvtx_range(name: str):
    try:
        import torch
        torch.cuda.nvtx.range_push(name)
        pushed = True
    except Exception:  # noqa: BLE001 - NVTX is best effort (CPU-only hosts)
        pushed = False
    try:
        yield
    finally:
        if pushed:
            import torch
            torch.cuda.nvtx.range_pop()
