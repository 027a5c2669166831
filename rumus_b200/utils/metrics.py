"""Observability: JSONL metrics sink per rank, device-side timers, NVTX ranges.

The reference has none of this beyond ``eprintln!`` in the server and ``Trainer::epoch_avg_loss``
(rumus/src/train.rs:78-85)."""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Optional

import torch


class MetricsLogger:
    """Appends one JSON object per ``log`` call to ``{dir}/metrics-rank{r}.jsonl``."""

    def __init__(self, directory: Optional[str], rank: int = 0):
        self.path = None
        if directory:
            os.makedirs(directory, exist_ok=True)
            self.path = os.path.join(directory, f"metrics-rank{rank}.jsonl")
        self.rank = rank

    def log(self, **kv) -> dict:
        rec = {"ts": time.time(), "rank": self.rank}
        for k, v in kv.items():
            if isinstance(v, torch.Tensor):
                v = v.item() if v.numel() == 1 else v.tolist()
            rec[k] = v
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        return rec


class DeviceTimer:
    """CUDA-event timer on the current stream (wall clock on CPU)."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        self.t0 = None

    def __enter__(self):
        if self.cuda:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.e0.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self.e1.record()
            self.e1.synchronize()
            self.ms = self.e0.elapsed_time(self.e1)
        else:
            self.ms = (time.perf_counter() - self.t0) * 1e3
        return False


_NVTX_ON = os.environ.get("RB_NVTX", "0") == "1"


def enable_tracing(on: bool = True) -> None:
    """Turns the NVTX ranges of the fused paths / pipeline / serving phases on or off (default:
    env ``RB_NVTX=1``)."""
    global _NVTX_ON
    _NVTX_ON = on


@contextlib.contextmanager
def trace_range(name: str):
    """NVTX range around a fused path or scheduler phase (shows up in profiler timelines).  Off by
    default so that the hot path pays nothing; no-op without CUDA."""
    if _NVTX_ON and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def peak_memory_gb() -> float:
    return torch.cuda.max_memory_allocated() / 2 ** 30 if torch.cuda.is_available() else 0.0


def kernel_breakdown(step_fn, steps: int = 2, top: int = 25):
    """Per-kernel device time of ``steps`` calls of ``step_fn`` (torch profiler, CUDA activities).

    Returns ``{"kernel_ms_per_step", "launches_per_step", "span_ms_per_step", "busy_fraction",
    "kernels": [[name, ms_per_step, launches_per_step], ...]}``.  Kernel durations measured under
    the profiler serve to rank kernels against each other; throughput numbers are always taken
    without it (CUDA events around unprofiled steps).
    """
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step_fn()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    agg = collections.defaultdict(lambda: [0.0, 0])
    for e in ev:
        agg[e.name][0] += e.device_time
        agg[e.name][1] += 1
    total = sum(v[0] for v in agg.values())
    span = (max(e.time_range.end for e in ev) - min(e.time_range.start for e in ev)) if ev else 0.0
    rows = [[name[:120], t / steps / 1e3, n / steps]
            for name, (t, n) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:top]]
    return {"kernel_ms_per_step": total / steps / 1e3,
            "launches_per_step": sum(v[1] for v in agg.values()) / steps,
            "span_ms_per_step": span / steps / 1e3,
            "busy_fraction": (total / span) if span else 0.0,
            "kernels": rows}
