"""Request-level scheduler of a replica pool: routing, admission, retries, metrics.

Every submitted prompt becomes an asyncio task that (1) asks the routing function for a
worker, (2) waits -- 5 ms at a time -- until that worker is below its concurrency limit,
(3) calls the worker, and (4) records what happened. A background loop polls the workers'
engine statistics twice a second and lets the concurrency function move the per-worker limits.

Routing functions and the limit controller follow the reference's semantics
(arctic_inference/server/scheduler.py:58-160): least loaded; prefix affinity over a ring of
the available workers with an 85 % load threshold and spill to the next ring position; strict
affinity that never spills; and a controller that grows limits while KV-cache utilisation is
below 90 %, backs off above 95 % or when the engine queues, and probes occasionally in between.
"""

from __future__ import annotations

import asyncio
import logging
import random
import time
import zlib
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence

from .metrics import (BoundedRing, ConcurrencyHistory, RequestRecord, WorkerMetricsCollector)

logger = logging.getLogger(__name__)

BACKOFF_S = 0.005
POLL_S = 0.5
PREFIX_LOAD_THRESHOLD = 0.85


@dataclass
class PendingRequest:
    id: int
    prompt: Any
    sampling_params: dict
    future: asyncio.Future
    prefix_hash: Optional[int] = None
    strict: bool = False
    routing_key: Optional[str] = None
    created_at: float = field(default_factory=time.time)
    worker_idx: Optional[int] = None
    retries: int = 0


@dataclass
class WorkerSlot:
    worker: Any
    concurrency_limit: int
    active_requests: int = 0
    available: bool = True
    latest_cache_utilization: float = 0.0
    running_reqs: int = 0
    waiting_reqs: int = 0
    tasks: set = field(default_factory=set)


def stable_hash(key) -> int:
    """Process-independent hash (Python's ``hash`` of a str changes between runs, which would
    move every conversation to another replica after a restart)."""
    if isinstance(key, str):
        data = key.encode()
    else:
        data = b",".join(str(int(t)).encode() for t in key)
    return zlib.crc32(data)


def _candidates(workers: Sequence[WorkerSlot]) -> list[int]:
    return [i for i, w in enumerate(workers) if w.available and w.concurrency_limit > 0]


def least_loaded_routing(req: PendingRequest, workers: Sequence[WorkerSlot]) -> int:
    cand = _candidates(workers) or list(range(len(workers)))
    return min(cand, key=lambda i: workers[i].active_requests / max(workers[i].concurrency_limit, 1))


def prefix_affinity_routing(req: PendingRequest, workers: Sequence[WorkerSlot]) -> int:
    cand = _candidates(workers)
    if not cand or req.prefix_hash is None:
        return least_loaded_routing(req, workers)
    for off in range(len(cand)):
        i = cand[(req.prefix_hash + off) % len(cand)]
        if workers[i].active_requests < workers[i].concurrency_limit * PREFIX_LOAD_THRESHOLD:
            return i
    return least_loaded_routing(req, workers)


def strict_affinity_routing(req: PendingRequest, workers: Sequence[WorkerSlot]) -> int:
    cand = _candidates(workers)
    if not cand or req.prefix_hash is None:
        return least_loaded_routing(req, workers)
    return cand[req.prefix_hash % len(cand)]


def utilization_based_concurrency(workers: Sequence[WorkerSlot], rng: random.Random = random) -> list[int]:
    TARGET, HIGH, MAX_QUEUE = 0.90, 0.95, 2
    LO, HI = 8, 2048
    backoff = 1 if rng.random() < 0.3 else 0
    out = []
    for w in workers:
        cur = max(w.concurrency_limit, LO)
        util = w.latest_cache_utilization
        if util == 0.0 and w.running_reqs == 0 and w.waiting_reqs == 0:
            # no reading yet (engine idle or statistics not in): follow the offered load
            new = max(LO, int(w.active_requests * 0.95)) if w.active_requests > 64 else \
                min(max(LO, int(w.active_requests * 1.5)), HI)
        elif util > HIGH or w.waiting_reqs > MAX_QUEUE:
            new = cur - backoff
        elif util < TARGET:
            new = cur + 2 + int(max(0.0, TARGET - util) * 10) if w.active_requests >= cur - 2 else cur
        else:
            probe = w.active_requests >= cur and w.waiting_reqs == 0 and rng.random() < 0.1
            new = cur + 1 if probe else cur
        out.append(max(LO, min(new, HI)))
    return out


def fixed_concurrency(limit: int) -> Callable:
    return lambda workers: [limit] * len(workers)


class Scheduler:
    def __init__(self, workers: Sequence[Any], routing_fn: Callable = prefix_affinity_routing,
                 concurrency_fn: Optional[Callable] = utilization_based_concurrency,
                 initial_limit: int = 64, max_retries: int = 2, poll_interval: float = POLL_S):
        self.workers: list[WorkerSlot] = [WorkerSlot(w, initial_limit) for w in workers]
        self.routing_fn = routing_fn
        self.concurrency_fn = concurrency_fn
        self.initial_limit = initial_limit
        self.max_retries = max_retries
        self.poll_interval = poll_interval
        self.records = BoundedRing()
        self.collectors = [WorkerMetricsCollector(i) for i in range(len(self.workers))]
        self.history = ConcurrencyHistory()
        self._next_id = 0
        self._paused = False
        self._tasks: set = set()
        self._poll_task: Optional[asyncio.Task] = None
        self._closed = False

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> None:
        if self._poll_task is None:
            self._poll_task = asyncio.ensure_future(self._poll_loop())

    async def close(self) -> None:
        self._closed = True
        if self._poll_task is not None:
            self._poll_task.cancel()
            try:
                await self._poll_task
            except (asyncio.CancelledError, Exception):  # noqa: BLE001
                pass
            self._poll_task = None
        for t in list(self._tasks):
            t.cancel()
        if self._tasks:
            await asyncio.gather(*self._tasks, return_exceptions=True)

    def add_worker(self, worker) -> int:
        self.workers.append(WorkerSlot(worker, self.initial_limit))
        self.collectors.append(WorkerMetricsCollector(len(self.workers) - 1))
        return len(self.workers) - 1

    def remove_worker(self, idx: int):
        slot = self.workers.pop(idx)
        self.collectors.pop(idx)
        for i, c in enumerate(self.collectors):
            c.worker_idx = i
        return slot.worker

    # ------------------------------------------------------------------ control
    def pause(self) -> None:
        self._paused = True

    def resume(self) -> None:
        self._paused = False

    @property
    def paused(self) -> bool:
        return self._paused

    @property
    def inflight(self) -> int:
        return len(self._tasks)

    async def drain(self, timeout: Optional[float] = None) -> None:
        """Wait until every request that was admitted has finished."""
        t0 = time.time()
        while self._tasks:
            if timeout is not None and time.time() - t0 > timeout:
                raise TimeoutError("%d requests still in flight" % len(self._tasks))
            await asyncio.sleep(BACKOFF_S)

    def mark_worker_unavailable(self, idx: int) -> None:
        self.workers[idx].available = False

    def mark_worker_available(self, idx: int) -> None:
        self.workers[idx].available = True

    async def cancel_worker_inflight(self, idx: int) -> int:
        """Cancel what a worker is running; the affected requests are retried elsewhere (or on
        the same worker once it is available again)."""
        try:
            return await self.workers[idx].worker.cancel_inflight()
        except Exception as e:  # noqa: BLE001
            logger.warning("cancel on worker %d failed: %s", idx, e)
            return 0

    # ------------------------------------------------------------------ submission
    def _make(self, prompt, params, routing_key, strict) -> PendingRequest:
        if self._closed:
            raise RuntimeError("scheduler closed")
        if self._paused:
            raise RuntimeError("scheduler is paused")
        self._next_id += 1
        key = routing_key if routing_key is not None else prompt
        req = PendingRequest(self._next_id, prompt, dict(params or {}),
                             asyncio.get_running_loop().create_future(),
                             prefix_hash=stable_hash(key), strict=strict, routing_key=routing_key)
        t = asyncio.ensure_future(self._process(req))
        self._tasks.add(t)
        t.add_done_callback(self._tasks.discard)
        return req

    async def submit(self, prompt, sampling_params=None, routing_key=None, strict=False) -> dict:
        return await self._make(prompt, sampling_params, routing_key, strict).future

    async def submit_batch(self, prompts, sampling_params=None, routing_key=None, strict=False) -> list:
        if routing_key is None or isinstance(routing_key, str):
            keys = [routing_key] * len(prompts)
        else:
            if len(routing_key) != len(prompts):
                raise ValueError("got %d routing keys for %d prompts" % (len(routing_key), len(prompts)))
            keys = list(routing_key)
        reqs = [self._make(p, sampling_params, k, strict) for p, k in zip(prompts, keys)]
        return list(await asyncio.gather(*[r.future for r in reqs]))

    async def _process(self, req: PendingRequest) -> None:
        last_err: Optional[BaseException] = None
        dispatched = req.created_at
        idx = -1
        while req.retries <= self.max_retries:
            # ---- route and wait for a slot
            while True:
                if not self.workers:
                    last_err = RuntimeError("no workers")
                    break
                fn = strict_affinity_routing if req.strict else self.routing_fn
                idx = fn(req, self.workers)
                slot = self.workers[idx]
                if slot.available and slot.active_requests < slot.concurrency_limit:
                    break
                await asyncio.sleep(BACKOFF_S)
            if not self.workers:
                break
            slot.active_requests += 1
            req.worker_idx = idx
            dispatched = time.time()
            try:
                res = await slot.worker.generate(req.prompt, req.sampling_params,
                                                 routing_key=req.routing_key)
                self.records.append(RequestRecord(
                    req.id, idx, req.created_at, dispatched, time.time(),
                    int(res.get("prompt_len", 0)), int(res.get("generation_len", 0)),
                    int(res.get("prefix_cache_len", 0)), res.get("finish_reason"), None, req.retries))
                if not req.future.done():
                    req.future.set_result(res)
                return
            except asyncio.CancelledError:
                if not req.future.done():
                    req.future.set_exception(RuntimeError("request cancelled"))
                raise
            except Exception as e:  # noqa: BLE001 - retried or reported below
                last_err = e
                req.retries += 1
                if isinstance(e, (ConnectionError, OSError)):
                    slot.available = False      # the health monitor decides when it returns
                logger.info("request %d failed on worker %d (%s); retry %d", req.id, idx, e, req.retries)
            finally:
                slot.active_requests -= 1
        self.records.append(RequestRecord(req.id, idx, req.created_at, dispatched, time.time(),
                                          error=str(last_err), retries=req.retries))
        if not req.future.done():
            req.future.set_exception(last_err if isinstance(last_err, RuntimeError)
                                     else RuntimeError(str(last_err)))

    # ------------------------------------------------------------------ statistics
    async def poll_once(self) -> None:
        async def one(i: int, slot: WorkerSlot) -> None:
            try:
                st = await asyncio.wait_for(slot.worker.get_stats(), timeout=5)
            except Exception:  # noqa: BLE001
                return
            slot.latest_cache_utilization = float(st.get("kv_cache_usage", 0.0))
            slot.running_reqs = int(st.get("running", 0))
            slot.waiting_reqs = int(st.get("waiting", 0))
            self.collectors[i].observe(st, slot.concurrency_limit, slot.active_requests)

        await asyncio.gather(*[one(i, s) for i, s in enumerate(self.workers)])
        if self.concurrency_fn is not None and self.workers:
            for slot, lim in zip(self.workers, self.concurrency_fn(self.workers)):
                slot.concurrency_limit = lim
            self.history.record([w.concurrency_limit for w in self.workers])

    async def _poll_loop(self) -> None:
        while True:
            await asyncio.sleep(self.poll_interval)
            try:
                await self.poll_once()
            except Exception as e:  # noqa: BLE001
                logger.warning("statistics poll failed: %s", e)

    def drain_metrics(self) -> dict:
        from dataclasses import asdict
        return {"requests": [asdict(r) for r in self.records.drain()],
                "replicas": [s for c in self.collectors for s in c.drain()],
                "concurrency": self.history.drain()}
