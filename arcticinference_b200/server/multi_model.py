"""Several models on one machine: a :class:`Driver` owns the GPUs and one
:class:`ReplicaPool` per model.

Policy (reference: arctic_inference/server/multi_model.py:48-133): GPUs are shared evenly.
Loading a model without an explicit replica count first shrinks the pools that hold more
than their new share, then starts the newcomer with its share; shutting a model down lets
the remaining pools grow back in the background. The driver has the pool's interface with
``model_id`` selecting the pool, so the REST layer works with either.
"""

from __future__ import annotations

import asyncio
import logging
import uuid
from typing import Callable, Optional

from .config import ServerModelConfig
from .replica_pool import GpuAllocator, ReplicaPool

logger = logging.getLogger(__name__)


class Driver:
    def __init__(self, worker_factory: Optional[Callable] = None, gpu_ids: Optional[list] = None,
                 **pool_kwargs):
        self.worker_factory = worker_factory
        self.allocator = GpuAllocator(gpu_ids)
        self.pool_kwargs = pool_kwargs
        self._pools: dict[str, ReplicaPool] = {}
        self._scale_tasks: dict[str, asyncio.Task] = {}

    # ------------------------------------------------------------------ shares
    @property
    def total_gpus(self) -> int:
        return self.allocator.total

    def even_share(self, per_replica: dict[str, int]) -> dict[str, int]:
        """Replicas per model when every model gets total/len(models) GPUs."""
        if not per_replica:
            return {}
        share = self.total_gpus // len(per_replica)
        out = {}
        for mid, g in per_replica.items():
            n = share // g
            if n == 0:
                raise RuntimeError("not enough GPUs for %r: a replica needs %d but the share is %d "
                                   "(%d GPUs / %d models)" % (mid, g, share, self.total_gpus,
                                                              len(per_replica)))
            out[mid] = n
        return out

    def _pool(self, model_id: Optional[str]) -> ReplicaPool:
        if model_id is None:
            if len(self._pools) == 1:
                return next(iter(self._pools.values()))
            raise ValueError("model_id is required when several models are loaded")
        if model_id not in self._pools:
            raise KeyError("unknown model_id %r; loaded: %s" % (model_id, sorted(self._pools)))
        return self._pools[model_id]

    def _rebalance_up(self) -> None:
        plan = self.even_share({m: p.gpus_per_replica for m, p in self._pools.items()})
        for mid, pool in self._pools.items():
            if plan[mid] > pool.num_replicas:
                old = self._scale_tasks.get(mid)
                if old is not None and not old.done():
                    old.cancel()
                logger.info("scaling %r up to %d replicas in the background", mid, plan[mid])
                self._scale_tasks[mid] = asyncio.ensure_future(pool.scale_up(plan[mid]))

    # ------------------------------------------------------------------ lifecycle
    async def initialize(self, config: ServerModelConfig, model_id: Optional[str] = None,
                         num_replicas: Optional[int] = None) -> int:
        if isinstance(config, dict):
            config = ServerModelConfig(**config)
        model_id = model_id or uuid.uuid4().hex[:8]
        if model_id in self._pools:
            raise ValueError("model_id %r is already loaded" % model_id)
        if num_replicas is None:
            per = {m: p.gpus_per_replica for m, p in self._pools.items()}
            per[model_id] = config.gpus_per_replica or config.world_size
            plan = self.even_share(per)
            for mid, pool in self._pools.items():
                t = self._scale_tasks.pop(mid, None)
                if t is not None and not t.done():
                    t.cancel()
                if plan[mid] < pool.num_replicas:
                    logger.info("shrinking %r: %d -> %d replicas", mid, pool.num_replicas, plan[mid])
                    await pool.scale_down(plan[mid])
            num_replicas = plan[model_id]
        pool = ReplicaPool(worker_factory=self.worker_factory, allocator=self.allocator,
                           base_port=29600 + 512 * len(self._pools), **self.pool_kwargs)
        n = await pool.initialize(config, model_id=model_id, num_replicas=num_replicas)
        self._pools[model_id] = pool
        return n

    async def shutdown(self, model_id: Optional[str] = None) -> None:
        if model_id is None:
            for t in self._scale_tasks.values():
                t.cancel()
            self._scale_tasks = {}
            await asyncio.gather(*[p.shutdown() for p in self._pools.values()])
            self._pools = {}
            return
        pool = self._pool(model_id)
        t = self._scale_tasks.pop(model_id, None)
        if t is not None and not t.done():
            t.cancel()
        await pool.shutdown()
        del self._pools[model_id]
        if self._pools:
            self._rebalance_up()

    async def wait_scaling(self) -> None:
        ts = [t for t in self._scale_tasks.values() if not t.done()]
        if ts:
            await asyncio.gather(*ts, return_exceptions=True)

    # ------------------------------------------------------------------ routed calls
    async def generate(self, prompts, sampling_params=None, model_id=None, routing_key=None,
                       strict: bool = False) -> list:
        return await self._pool(model_id).generate(prompts, sampling_params, routing_key=routing_key,
                                                   strict=strict)

    async def sleep(self, model_id=None, level: int = 1) -> dict:
        return await self._pool(model_id).sleep(level=level)

    async def wake_up(self, model_id=None, tags=None) -> dict:
        return await self._pool(model_id).wake_up(tags=tags)

    async def reset_prefix_cache(self, model_id=None) -> dict:
        return await self._pool(model_id).reset_prefix_cache()

    async def get_weights_info_async(self, model_id=None) -> list:
        return await self._pool(model_id).get_weights_info_async()

    async def get_spec_weights_info_async(self, model_id=None) -> list:
        return await self._pool(model_id).get_spec_weights_info_async()

    async def sync_weights(self, model_id=None, **kw) -> dict:
        return await self._pool(model_id).sync_weights(**kw)

    async def sync_spec_weights(self, model_id=None, **kw) -> dict:
        return await self._pool(model_id).sync_spec_weights(**kw)

    async def close_weight_sync(self, model_id=None) -> dict:
        return await self._pool(model_id).close_weight_sync()

    async def drain_metrics(self, model_id=None) -> dict:
        if model_id is not None:
            return await self._pool(model_id).drain_metrics()
        return {m: await p.drain_metrics() for m, p in self._pools.items()}

    async def get_status(self) -> dict:
        return {"total_gpus": self.total_gpus, "free_gpus": len(self.allocator.free),
                "models": {m: await p.get_status() for m, p in self._pools.items()}}
