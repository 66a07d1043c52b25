"""Lightweight tracing of the engine's host loop and device steps.

* ``trace_range(name)``: NVTX range (shows up in Nsight tools) plus, when a ``Tracer`` is
  active, a host-side interval for the Chrome trace;
* ``StepTimer``: CUDA-event timing of engine steps on the launching stream; in a multi-GPU
  engine the reported step time is the maximum over ranks (``reduce_max``);
* ``Tracer``: collects host intervals and writes ``chrome://tracing`` JSON.

The reference only marks its sample / draft / bookkeeping phases with profiler ranges
(arctic_inference/vllm/model_runner.py:1295-1676); it has no timers of its own. Tracing is off
unless ``ARCTIC_B200_TRACE=1`` or a tracer is installed explicitly, and costs one attribute
check per range when off.
"""

from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from typing import Optional

import torch

_active: Optional["Tracer"] = None
_nvtx = os.environ.get("ARCTIC_B200_TRACE", "0") not in ("0", "", "false")


class Tracer:
    def __init__(self):
        self.events: list = []
        self._lock = threading.Lock()
        self.t0 = time.perf_counter()

    def add(self, name: str, start: float, end: float, args: Optional[dict] = None) -> None:
        with self._lock:
            self.events.append({"name": name, "ph": "X", "pid": os.getpid(),
                                "tid": threading.get_ident() % 100000,
                                "ts": (start - self.t0) * 1e6, "dur": (end - start) * 1e6,
                                "args": args or {}})

    def dump(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)

    def totals(self) -> dict:
        out: dict = {}
        for e in self.events:
            tot, n = out.get(e["name"], (0.0, 0))
            out[e["name"]] = (tot + e["dur"] / 1e3, n + 1)
        return out

    def __enter__(self):
        install(self)
        return self

    def __exit__(self, *exc):
        install(None)


def install(tracer: Optional[Tracer]) -> None:
    global _active
    _active = tracer


def enable_nvtx(on: bool = True) -> None:
    global _nvtx
    _nvtx = on


@contextlib.contextmanager
def trace_range(name: str, **args):
    if _active is None and not _nvtx:
        yield
        return
    pushed = False
    if _nvtx and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        pushed = True
    t0 = time.perf_counter()
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()
        if _active is not None:
            _active.add(name, t0, time.perf_counter(), args)


class StepTimer:
    """Device time of consecutive steps: ``start()`` / ``stop()`` bracket a step with CUDA
    events on the current stream; ``times_ms()`` synchronises once and returns all durations."""

    def __init__(self, device=None):
        self.device = device
        self._pairs: list = []
        self._open = None

    def start(self) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._open = e

    def stop(self) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._pairs.append((self._open, e))
        self._open = None

    def times_ms(self) -> list:
        if self._pairs:
            self._pairs[-1][1].synchronize()
        return [a.elapsed_time(b) for a, b in self._pairs]

    def reduce_max(self, comm=None) -> list:
        """Per-step maximum over the ranks of ``comm`` (None: this rank's own times)."""
        t = self.times_ms()
        if comm is None or comm.world == 1:
            return t
        import torch.distributed as dist
        x = torch.tensor(t, dtype=torch.float64, device=self.device or "cuda")
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return x.tolist()
