"""Replica pool: N independent engines of one model behind one scheduler.

Covers the life cycle the reference implements with Ray actors and placement groups
(arctic_inference/server/replica_pool.py:165-283 initialise, :384-452 scale, :462-551
sleep / staged wake, :630-753 weight sync with drain / skip / hotswap, :939-982 health monitor
and restart): here a replica is a :class:`ProcessWorker` (child processes pinned to the
replica's GPUs through ``CUDA_VISIBLE_DEVICES``) or any object with the worker interface
(``worker_factory``: in-process engines and test fakes).
"""

from __future__ import annotations

import asyncio
import logging
import time
from typing import Callable, Optional

from .config import ServerModelConfig
from .scheduler import Scheduler, prefix_affinity_routing, utilization_based_concurrency
from .worker import ProcessWorker

logger = logging.getLogger(__name__)


def visible_gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:  # noqa: BLE001
        return 0


class GpuAllocator:
    """Free list of GPU ids shared by the pools of one server."""

    def __init__(self, gpu_ids: Optional[list] = None):
        self.all = list(gpu_ids) if gpu_ids is not None else list(range(visible_gpu_count()))
        self.free = list(self.all)

    @property
    def total(self) -> int:
        return len(self.all)

    def acquire(self, n: int) -> Optional[list]:
        if not self.all:
            return None            # CPU-only host: replicas are not pinned
        if n > len(self.free):
            raise RuntimeError("replica needs %d GPUs but only %d of %d are free" %
                               (n, len(self.free), len(self.all)))
        got, self.free = self.free[:n], self.free[n:]
        return got

    def release(self, ids: Optional[list]) -> None:
        if ids:
            self.free = sorted(set(self.free) | set(ids))


class ReplicaPool:
    def __init__(self, worker_factory: Optional[Callable] = None, gpu_ids: Optional[list] = None,
                 allocator: Optional[GpuAllocator] = None,
                 routing_fn: Callable = prefix_affinity_routing,
                 concurrency_fn: Optional[Callable] = utilization_based_concurrency,
                 health_interval: float = 0.0, base_port: int = 29600):
        self.worker_factory = worker_factory
        self.allocator = allocator or GpuAllocator(gpu_ids)
        self.routing_fn = routing_fn
        self.concurrency_fn = concurrency_fn
        self.health_interval = health_interval      # 0 = monitor off (the reference's default)
        self.base_port = base_port
        self._config: Optional[ServerModelConfig] = None
        self._model_id: Optional[str] = None
        self._workers: list = []
        self._worker_gpus: list = []
        self._scheduler: Optional[Scheduler] = None
        self._sleeping = False
        self._lock = asyncio.Lock()
        self._health_task: Optional[asyncio.Task] = None
        self._updating_workers: set = set()
        self._next_worker_id = 0
        self.restarts = 0

    # ------------------------------------------------------------------ properties
    @property
    def config(self) -> ServerModelConfig:
        if self._config is None:
            raise RuntimeError("ReplicaPool not initialized")
        return self._config

    @property
    def model_id(self) -> Optional[str]:
        return self._model_id

    @property
    def tp_size(self) -> int:
        return self.config.world_size

    @property
    def num_replicas(self) -> int:
        return len(self._workers)

    @property
    def sleeping(self) -> bool:
        return self._sleeping

    def _check_model_id(self, model_id: Optional[str]) -> None:
        if model_id is not None and self._model_id is not None and model_id != self._model_id:
            raise ValueError("model_id %r does not match the loaded model %r" % (model_id, self._model_id))

    # ------------------------------------------------------------------ workers
    @property
    def gpus_per_replica(self) -> int:
        return self.config.gpus_per_replica or self.config.world_size

    async def _spawn(self, slot: int):
        wid = self._next_worker_id
        self._next_worker_id += 1
        gpus = self.allocator.acquire(self.gpus_per_replica)
        try:
            if self.worker_factory is not None:
                w = self.worker_factory(wid)
            else:
                w = ProcessWorker(wid, gpus, master_port=self.base_port + 16 * wid)
            await w.initialize(self.config)
        except BaseException:
            self.allocator.release(gpus)
            raise
        return w, gpus

    async def initialize(self, config: ServerModelConfig, model_id: Optional[str] = None,
                         num_replicas: Optional[int] = None) -> int:
        async with self._lock:
            if self._workers:
                raise RuntimeError("pool already initialized; shut it down first")
            if isinstance(config, dict):
                config = ServerModelConfig(**config)
            self._config = config
            self._model_id = model_id or config.model
            if num_replicas is None:
                num_replicas = max(1, len(self.allocator.free) // self.gpus_per_replica)
            res = await asyncio.gather(*[self._spawn(i) for i in range(num_replicas)],
                                       return_exceptions=True)
            bad = [r for r in res if isinstance(r, BaseException)]
            if bad:
                for r in res:
                    if not isinstance(r, BaseException):
                        await r[0].shutdown()
                        self.allocator.release(r[1])
                self._config = None
                self._model_id = None
                raise bad[0]
            self._workers = [w for w, _ in res]
            self._worker_gpus = [g for _, g in res]
            self._scheduler = Scheduler(self._workers, self.routing_fn, self.concurrency_fn)
            self._scheduler.start()
            self._sleeping = False
            if self.health_interval > 0:
                self._health_task = asyncio.ensure_future(self._monitor_health())
            return len(self._workers)

    async def shutdown(self, model_id: Optional[str] = None) -> None:
        self._check_model_id(model_id)
        async with self._lock:
            if self._health_task is not None:
                self._health_task.cancel()
                self._health_task = None
            if self._scheduler is not None:
                await self._scheduler.close()
                self._scheduler = None
            await asyncio.gather(*[w.shutdown() for w in self._workers], return_exceptions=True)
            for g in self._worker_gpus:
                self.allocator.release(g)
            self._workers, self._worker_gpus = [], []
            self._config = None
            self._model_id = None
            self._sleeping = False

    # ------------------------------------------------------------------ serving
    async def generate(self, prompts, sampling_params: Optional[dict] = None,
                       model_id: Optional[str] = None, routing_key=None, strict: bool = False) -> list:
        self._check_model_id(model_id)
        if self._scheduler is None:
            raise RuntimeError("ReplicaPool not initialized")
        if self._sleeping:
            raise RuntimeError("Model is sleeping; call /wake_up first")
        params = sampling_params or {}
        single = isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int))
        if single:
            key = routing_key
            if isinstance(routing_key, (list, tuple)):
                if len(routing_key) != 1:
                    raise ValueError("got %d routing keys for a single prompt" % len(routing_key))
                key = routing_key[0]
            return [await self._scheduler.submit(prompts, params, routing_key=key, strict=strict)]
        return await self._scheduler.submit_batch(list(prompts), params, routing_key=routing_key,
                                                  strict=strict)

    # ------------------------------------------------------------------ scaling
    async def scale_down(self, target_count: int) -> None:
        async with self._lock:
            while len(self._workers) > max(target_count, 0):
                idx = len(self._workers) - 1
                self._scheduler.mark_worker_unavailable(idx)
                # let the replica finish what it has
                while self._scheduler.workers[idx].active_requests:
                    await asyncio.sleep(0.005)
                w = self._scheduler.remove_worker(idx)
                self._workers.pop(idx)
                await w.shutdown()
                self.allocator.release(self._worker_gpus.pop(idx))

    async def scale_up(self, target_count: int) -> None:
        async with self._lock:
            n0 = len(self._workers)
            if target_count <= n0:
                return
            res = await asyncio.gather(*[self._spawn(i) for i in range(n0, target_count)])
            for w, g in res:
                if self._sleeping:
                    await w.sleep(1)
                self._workers.append(w)
                self._worker_gpus.append(g)
                self._scheduler.add_worker(w)

    # ------------------------------------------------------------------ sleep / wake
    async def sleep(self, model_id: Optional[str] = None, level: int = 1) -> dict:
        self._check_model_id(model_id)
        async with self._lock:
            if self._sleeping:
                return {"status": "sleeping", "level": level}
            t0 = time.time()
            self._scheduler.pause()
            await self._scheduler.drain()
            await asyncio.gather(*[w.sleep(level) for w in self._workers])
            self._sleeping = True
            return {"status": "sleeping", "level": level, "seconds": time.time() - t0}

    async def wake_up(self, model_id: Optional[str] = None, tags: Optional[list] = None) -> dict:
        """``tags = ["weights"]`` restores only the weights (a weight sync can then run before
        memory is spent on the KV cache); a later call with ``["kv_cache"]`` (or no tags)
        completes the wake-up and resumes serving."""
        self._check_model_id(model_id)
        async with self._lock:
            if not self._sleeping:
                return {"status": "awake"}
            t0 = time.time()
            res = await asyncio.gather(*[w.wake_up(tags) for w in self._workers], return_exceptions=True)
            bad = [r for r in res if isinstance(r, BaseException)]
            if bad:
                raise RuntimeError("wake_up failed on %d replicas: %s" % (len(bad), bad[0]))
            final = tags is None or "kv_cache" in tags
            if final:
                self._sleeping = False
                self._scheduler.resume()
            return {"status": "awake" if final else "weights_ready", "tags": tags,
                    "seconds": time.time() - t0}

    async def reset_prefix_cache(self, model_id: Optional[str] = None) -> dict:
        self._check_model_id(model_id)
        await asyncio.gather(*[w.reset_prefix_cache() for w in self._workers])
        return {"status": "ok", "replicas": len(self._workers)}

    # ------------------------------------------------------------------ status / metrics
    async def get_status(self) -> dict:
        if self._config is None:
            return {"initialized": False}
        sched = self._scheduler
        return {"initialized": True, "model_id": self._model_id, "model": self._config.model,
                "num_replicas": len(self._workers), "sleeping": self._sleeping,
                "paused": sched.paused, "inflight": sched.inflight, "restarts": self.restarts,
                "workers": [{"idx": i, "status": getattr(w.status, "value", str(w.status)),
                             "gpus": self._worker_gpus[i], "available": s.available,
                             "active_requests": s.active_requests,
                             "concurrency_limit": s.concurrency_limit,
                             "kv_cache_usage": s.latest_cache_utilization}
                            for i, (w, s) in enumerate(zip(self._workers, sched.workers))]}

    async def drain_metrics(self, model_id: Optional[str] = None) -> dict:
        self._check_model_id(model_id)
        if self._scheduler is None:
            return {"requests": [], "replicas": [], "concurrency": []}
        return self._scheduler.drain_metrics()

    async def compute_weight_norm(self, model_id: Optional[str] = None) -> dict:
        self._check_model_id(model_id)
        norms = await asyncio.gather(*[w.compute_weight_norm() for w in self._workers])
        return {"norms": list(norms)}

    # ------------------------------------------------------------------ weights
    async def get_weights_info_async(self, model_id: Optional[str] = None) -> list:
        self._check_model_id(model_id)
        if not self._workers:
            raise RuntimeError("ReplicaPool not initialized")
        return await self._workers[0].weights_info()

    async def get_spec_weights_info_async(self, model_id: Optional[str] = None) -> list:
        self._check_model_id(model_id)
        if not self._workers:
            raise RuntimeError("ReplicaPool not initialized")
        return await self._workers[0].spec_weights_info()

    def _groups(self, groups, master_addr, master_port, world_size) -> dict:
        if groups is None:
            if master_addr is None or master_port is None:
                raise ValueError("provide 'groups' or master_addr / master_port")
            groups = [{"group_id": 0, "master_addr": master_addr, "master_port": master_port,
                       "world_size": world_size or 1 + self.num_replicas * self.tp_size,
                       "replica_ids": list(range(self.num_replicas))}]
        tp = self.tp_size
        plan = {}
        for g in groups:
            g = g if isinstance(g, dict) else g.model_dump()
            for rid in g["replica_ids"]:
                if not 0 <= rid < self.num_replicas:
                    raise ValueError("replica id %d out of range" % rid)
                # every (replica, rank) pair gets a private two-party channel to the sender
                plan[rid] = {"master_addr": g["master_addr"], "master_port": g["master_port"] + rid * tp}
        return plan

    async def _sync(self, method: str, groups, bucket_size, strategy, extra: dict, model_id,
                    master_addr, master_port, world_size) -> dict:
        self._check_model_id(model_id)
        if self._scheduler is None:
            raise RuntimeError("ReplicaPool not initialized")
        if strategy not in ("drain", "skip", "hotswap"):
            raise ValueError("unknown strategy %r; use drain, skip or hotswap" % strategy)
        plan = self._groups(groups, master_addr, master_port, world_size)
        async with self._lock:
            t0 = time.time()
            sched = self._scheduler
            ids = sorted(plan)
            was_paused = sched.paused
            if strategy == "drain":
                sched.pause()
                await sched.drain()
            elif strategy == "skip":
                for i in ids:
                    sched.mark_worker_unavailable(i)
                await asyncio.gather(*[sched.cancel_worker_inflight(i) for i in ids])
            self._updating_workers = set(ids)
            try:
                res = await asyncio.gather(*[
                    getattr(self._workers[i], method)(bucket_size=bucket_size, **plan[i], **extra)
                    for i in ids], return_exceptions=True)
            finally:
                self._updating_workers = set()
                if strategy == "drain" and not was_paused and not self._sleeping:
                    sched.resume()
                elif strategy == "skip":
                    for i in ids:
                        sched.mark_worker_available(i)
            bad = [(i, r) for i, r in zip(ids, res) if isinstance(r, BaseException)]
            if bad:
                raise RuntimeError("weight sync failed on replica %d: %s" % bad[0])
            # cached prefixes were computed with the old weights
            await asyncio.gather(*[self._workers[i].reset_prefix_cache() for i in ids],
                                 return_exceptions=True)
            return {"status": "ok", "strategy": strategy, "replicas": ids, "seconds": time.time() - t0,
                    "results": list(res)}

    async def sync_weights(self, groups=None, bucket_size: int = 256 << 20, strategy: str = "hotswap",
                           engine_only: bool = False, direct_mode: bool = False, reverse: bool = False,
                           model_id=None, master_addr=None, master_port=None, world_size=None) -> dict:
        extra = {"engine_only": engine_only, "direct_mode": direct_mode, "reverse": reverse}
        return await self._sync("sync_weights", groups, bucket_size, strategy, extra, model_id,
                                master_addr, master_port, world_size)

    async def sync_spec_weights(self, groups=None, bucket_size: int = 256 << 20,
                                strategy: str = "hotswap", engine_only: bool = False,
                                reverse: bool = False, model_id=None, master_addr=None,
                                master_port=None, world_size=None) -> dict:
        extra = {"engine_only": engine_only, "reverse": reverse}
        return await self._sync("sync_spec_weights", groups, bucket_size, strategy, extra, model_id,
                                master_addr, master_port, world_size)

    async def sync_weights_ipc(self, key: str, model_id=None, strategy: str = "drain") -> dict:
        """Colocated trainer: weights are handed over through shared memory / CUDA IPC handles
        published under ``key`` (see weight_sync/ipc_engine.py)."""
        return await self._sync("sync_weights", [{"group_id": 0, "master_addr": "ipc://" + key,
                                                  "master_port": 0, "world_size": 0,
                                                  "replica_ids": list(range(self.num_replicas))}],
                                0, strategy, {}, model_id, None, None, None)

    async def close_weight_sync(self, model_id: Optional[str] = None) -> dict:
        self._check_model_id(model_id)
        res = await asyncio.gather(*[w.close_weight_sync() for w in self._workers],
                                   return_exceptions=True)
        return {"status": "ok", "closed": sum(int(r.get("closed", 0)) for r in res if isinstance(r, dict))}

    # ------------------------------------------------------------------ health
    async def check_health_once(self) -> list:
        """Probe every replica; restart the ones that do not answer. Returns restarted slots."""
        res = await asyncio.gather(*[w.health() for w in self._workers], return_exceptions=True)
        restarted = []
        for i, ok in enumerate(res):
            if ok is True or i in self._updating_workers:
                continue
            logger.warning("replica %d failed its health check (%r): restarting", i, ok)
            await self._restart_worker(i)
            restarted.append(i)
        return restarted

    async def _monitor_health(self) -> None:
        while True:
            await asyncio.sleep(self.health_interval)
            try:
                await self.check_health_once()
            except Exception as e:  # noqa: BLE001
                logger.warning("health monitor round failed: %s", e)

    async def _restart_worker(self, idx: int) -> None:
        sched = self._scheduler
        sched.mark_worker_unavailable(idx)
        old = self._workers[idx]
        try:
            await asyncio.wait_for(old.shutdown(), timeout=30)
        except Exception:  # noqa: BLE001
            pass
        self.allocator.release(self._worker_gpus[idx])
        self._worker_gpus[idx] = None
        w, g = await self._spawn(idx)
        if self._sleeping:
            await w.sleep(1)
        self._workers[idx] = w
        self._worker_gpus[idx] = g
        sched.workers[idx].worker = w
        sched.workers[idx].active_requests = 0
        sched.mark_worker_available(idx)
        self.restarts += 1
