"""Serving metrics: per-request records, per-replica snapshots, bounded rings, and the
history of concurrency limits.

Consumers *drain* the rings (each ``/metrics`` call returns what accumulated since the last
one), so nothing grows without bound on a long-running server
(reference: arctic_inference/server/metrics.py:53-120, :128-223, :283-342).
"""

from __future__ import annotations

import bisect
import threading
import time
from collections import deque
from dataclasses import asdict, dataclass
from typing import Any, Optional


@dataclass
class RequestRecord:
    request_id: int
    worker_idx: int
    created_at: float
    dispatched_at: float
    finished_at: float
    prompt_len: int = 0
    generation_len: int = 0
    prefix_cache_len: int = 0
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    retries: int = 0

    @property
    def queue_time(self) -> float:
        return self.dispatched_at - self.created_at

    @property
    def latency(self) -> float:
        return self.finished_at - self.created_at


@dataclass
class ReplicaSnapshot:
    worker_idx: int
    timestamp: float
    running: int = 0
    waiting: int = 0
    kv_cache_usage: float = 0.0
    prompt_tokens: int = 0
    generation_tokens: int = 0
    draft_tokens: int = 0
    accepted_tokens: int = 0
    concurrency_limit: int = 0
    active_requests: int = 0


class BoundedRing:
    """Thread-safe ring of the most recent ``maxlen`` items; ``drain`` empties it. Pickles as
    its contents (locks do not travel between processes)."""

    def __init__(self, maxlen: int = 65536):
        self.maxlen = maxlen
        self._d: deque = deque(maxlen=maxlen)
        self._lock = threading.Lock()
        self.dropped = 0

    def append(self, item) -> None:
        with self._lock:
            if len(self._d) == self.maxlen:
                self.dropped += 1
            self._d.append(item)

    def drain(self) -> list:
        with self._lock:
            out = list(self._d)
            self._d.clear()
            return out

    def __len__(self) -> int:
        return len(self._d)

    def __getstate__(self):
        with self._lock:
            return {"maxlen": self.maxlen, "items": list(self._d), "dropped": self.dropped}

    def __setstate__(self, st):
        self.maxlen = st["maxlen"]
        self._d = deque(st["items"], maxlen=self.maxlen)
        self._lock = threading.Lock()
        self.dropped = st["dropped"]


class WorkerMetricsCollector:
    """Turns a worker's engine statistics into ``ReplicaSnapshot`` rows, at most one per
    ``min_interval`` seconds."""

    def __init__(self, worker_idx: int, min_interval: float = 1.0, maxlen: int = 4096):
        self.worker_idx = worker_idx
        self.min_interval = min_interval
        self.ring = BoundedRing(maxlen)
        self._last = 0.0

    def observe(self, stats: dict, concurrency_limit: int = 0, active_requests: int = 0,
                now: Optional[float] = None) -> Optional[ReplicaSnapshot]:
        now = time.time() if now is None else now
        if now - self._last < self.min_interval:
            return None
        self._last = now
        snap = ReplicaSnapshot(
            self.worker_idx, now, int(stats.get("running", 0)), int(stats.get("waiting", 0)),
            float(stats.get("kv_cache_usage", 0.0)), int(stats.get("prompt_tokens", 0)),
            int(stats.get("generation_tokens", 0)), int(stats.get("draft_tokens", 0)),
            int(stats.get("accepted_tokens", 0)), concurrency_limit, active_requests)
        self.ring.append(snap)
        return snap

    def drain(self) -> list[dict]:
        return [asdict(s) for s in self.ring.drain()]


class ConcurrencyHistory:
    """Time series of (timestamp, limits per worker); ``at(t)`` answers what the limits were
    when a request was dispatched."""

    def __init__(self, maxlen: int = 8192):
        self._t: list[float] = []
        self._v: list[list[int]] = []
        self.maxlen = maxlen

    def record(self, limits: list[int], now: Optional[float] = None) -> None:
        now = time.time() if now is None else now
        if self._v and self._v[-1] == list(limits):
            return
        self._t.append(now)
        self._v.append(list(limits))
        if len(self._t) > self.maxlen:
            drop = len(self._t) - self.maxlen
            del self._t[:drop], self._v[:drop]

    def at(self, t: float) -> Optional[list[int]]:
        i = bisect.bisect_right(self._t, t) - 1
        return self._v[i] if i >= 0 else None

    def drain(self) -> list[dict]:
        out = [{"timestamp": t, "limits": v} for t, v in zip(self._t, self._v)]
        # keep the last point so that later lookups still resolve
        self._t, self._v = self._t[-1:], self._v[-1:]
        return out


def summarize(records: list[RequestRecord]) -> dict[str, Any]:
    """Aggregate view used by ``/status``."""
    ok = [r for r in records if r.error is None]
    if not ok:
        return {"count": len(records), "errors": len(records)}
    lat = sorted(r.latency for r in ok)
    pick = lambda q: lat[min(len(lat) - 1, int(q * len(lat)))]
    span = max(r.finished_at for r in ok) - min(r.created_at for r in ok)
    toks = sum(r.prompt_len + r.generation_len for r in ok)
    return {"count": len(records), "errors": len(records) - len(ok), "p50_latency": pick(0.5),
            "p99_latency": pick(0.99), "mean_queue_time": sum(r.queue_time for r in ok) / len(ok),
            "tokens_per_s": toks / span if span > 0 else 0.0}
