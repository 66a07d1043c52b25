"""Inference workers: one replica of one model.

``InferenceWorker`` hosts an :class:`AsyncLLM` in the current process. ``ProcessWorker`` is a
proxy with the same coroutine interface whose engine lives in child processes: one process
per GPU of the replica, rank 0 answering calls over a pipe, the other ranks following its
requests (see :mod:`arcticinference_b200.engine.async_llm`). The reference hosts its engine in
a Ray actor and fans calls out to tensor-parallel workers through ``collective_rpc``
(arctic_inference/server/worker.py:117-228, :414-513); no Ray is needed here.

States (reference :90-96, :275-390): UNINITIALIZED -> READY <-> SLEEPING, with WEIGHTS_READY
between a ``wake_up(tags=["weights"])`` and the ``wake_up(tags=["kv_cache"])`` that completes
it (weights can be synced while the KV cache is still released).
"""

from __future__ import annotations

import asyncio
import enum
import logging
import multiprocessing as mp
import os
import threading
import traceback
from typing import Any, Optional

logger = logging.getLogger(__name__)


class WorkerStatus(str, enum.Enum):
    UNINITIALIZED = "uninitialized"
    READY = "ready"
    SLEEPING = "sleeping"
    WEIGHTS_READY = "weights_ready"


class WorkerBase:
    def __init__(self, idx: int = 0):
        self.idx = idx
        self.status = WorkerStatus.UNINITIALIZED
        self.config = None

    async def initialize(self, config) -> None:
        raise NotImplementedError

    async def generate(self, prompt, sampling_params=None, request_id=None, routing_key=None) -> dict:
        raise NotImplementedError

    async def cancel_inflight(self) -> int:
        return 0

    async def get_stats(self) -> dict:
        return {}

    async def health(self) -> bool:
        return self.status is not WorkerStatus.UNINITIALIZED

    async def sleep(self, level: int = 1) -> None:
        raise NotImplementedError

    async def wake_up(self, tags=None) -> None:
        raise NotImplementedError

    async def reset_prefix_cache(self) -> None:
        pass

    async def weights_info(self) -> list[dict]:
        return []

    async def spec_weights_info(self) -> list[dict]:
        return []

    async def sync_weights(self, **kw) -> dict:
        raise NotImplementedError

    async def sync_spec_weights(self, **kw) -> dict:
        raise NotImplementedError

    async def close_weight_sync(self) -> dict:
        return {"closed": 0}

    async def compute_weight_norm(self) -> float:
        return 0.0

    async def shutdown(self) -> None:
        pass


def _result_dict(out, want_logprobs: bool, want_prompt_logprobs: bool) -> dict[str, Any]:
    c = out.outputs[0]
    d = {"text": c.text, "token_ids": list(c.token_ids), "finish_reason": c.finish_reason,
         "prompt_len": len(out.prompt_token_ids), "generation_len": len(c.token_ids),
         "prefix_cache_len": int(out.num_cached_tokens)}
    if len(out.outputs) > 1:
        d["samples"] = [{"index": o.index, "text": o.text, "token_ids": list(o.token_ids),
                         "finish_reason": o.finish_reason} for o in out.outputs]
    if want_logprobs:
        d["logprobs"] = c.logprobs
    if want_prompt_logprobs:
        d["prompt_logprobs"] = out.prompt_logprobs
    return d


class InferenceWorker(WorkerBase):
    """Engine in this process (rank 0 of the replica when it spans several GPUs)."""

    def __init__(self, idx: int = 0, device: Optional[str] = None):
        super().__init__(idx)
        self.device = device
        self.llm = None
        self._inflight: dict[str, asyncio.Task] = {}
        self._awake_tags: set = set()
        self._seq = 0

    async def initialize(self, config) -> None:
        from ..config import EngineArgs
        from ..engine.async_llm import AsyncLLM
        for k, v in (config.extra_env or {}).items():
            os.environ[k] = str(v)
        kw = config.to_engine_kwargs()
        loop = asyncio.get_running_loop()
        # engine construction loads weights and captures graphs: keep the event loop free
        self.llm = await loop.run_in_executor(
            None, lambda: AsyncLLM.from_engine_args(EngineArgs(**kw), device=self.device))
        self.config = config
        if self.llm.is_leader:
            self.llm.start()
        self.status = WorkerStatus.READY

    def run_follower(self) -> None:
        self.llm.run_follower()

    async def generate(self, prompt, sampling_params=None, request_id=None, routing_key=None) -> dict:
        if self.status is not WorkerStatus.READY:
            raise RuntimeError("worker %d is %s" % (self.idx, self.status.value))
        from ..engine.sampling_params import SamplingParams
        sp = dict(sampling_params or {})
        params = sp if isinstance(sp, SamplingParams) else SamplingParams(**sp)
        self._seq += 1
        rid = request_id or "w%d-%d" % (self.idx, self._seq)
        task = asyncio.ensure_future(self.llm.generate_final(prompt, params, rid, routing_key))
        self._inflight[rid] = task
        try:
            out = await task
        except asyncio.CancelledError:
            await self.llm.abort(rid)
            raise RuntimeError("request cancelled")
        finally:
            self._inflight.pop(rid, None)
        if out is None:
            raise RuntimeError("request cancelled")
        return _result_dict(out, params.logprobs is not None, params.prompt_logprobs is not None)

    async def cancel_inflight(self) -> int:
        tasks = list(self._inflight.values())
        for t in tasks:
            t.cancel()
        return len(tasks)

    async def get_stats(self) -> dict:
        if self.llm is None:
            return {}
        return await self.llm.get_stats()

    async def health(self) -> bool:
        return self.llm is not None and self.llm._dead is None

    async def sleep(self, level: int = 1) -> None:
        if self.status is WorkerStatus.SLEEPING:
            return
        await self.llm.sleep(level)
        self._awake_tags = set()
        self.status = WorkerStatus.SLEEPING

    async def wake_up(self, tags=None) -> None:
        if self.status is WorkerStatus.READY:
            return
        await self.llm.wake_up(list(tags) if tags else None)
        self._awake_tags |= set(tags) if tags else {"weights", "kv_cache"}
        if "kv_cache" in self._awake_tags:
            self.status = WorkerStatus.READY
        else:
            self.status = WorkerStatus.WEIGHTS_READY

    async def reset_prefix_cache(self) -> None:
        await self.llm.reset_prefix_cache()

    # ---- weights: executed on every rank's engine thread between two steps
    async def weights_info(self) -> list[dict]:
        from .weight_sync.receiver import engine_weights_info
        return await self.llm.apply(engine_weights_info)

    async def spec_weights_info(self) -> list[dict]:
        from .weight_sync.receiver import engine_spec_weights_info
        return await self.llm.apply(engine_spec_weights_info)

    async def sync_weights(self, **kw) -> dict:
        if self.status not in (WorkerStatus.READY, WorkerStatus.WEIGHTS_READY):
            raise RuntimeError("worker %d is %s; wake its weights first" % (self.idx, self.status.value))
        from .weight_sync.receiver import engine_sync_weights
        return await self.llm.apply(engine_sync_weights, kw)

    async def sync_spec_weights(self, **kw) -> dict:
        from .weight_sync.receiver import engine_sync_weights
        return await self.llm.apply(engine_sync_weights, dict(kw, target="speculator"))

    async def close_weight_sync(self) -> dict:
        from .weight_sync.receiver import engine_close_weight_sync
        return await self.llm.apply(engine_close_weight_sync)

    async def compute_weight_norm(self) -> float:
        from .weight_sync.utils import engine_weight_norm
        return await self.llm.apply(engine_weight_norm)

    async def shutdown(self) -> None:
        if self.llm is not None:
            await self.cancel_inflight()
            self.llm.shutdown()
            self.llm = None
        self.status = WorkerStatus.UNINITIALIZED


# ------------------------------------------------------------------------------------------
# subprocess hosting
# ------------------------------------------------------------------------------------------
def _child_main(conn, idx: int, rank: int, env: dict, config_json: str) -> None:
    os.environ.update(env)
    logging.basicConfig(level=logging.INFO)
    from .config import ServerModelConfig
    cfg = ServerModelConfig.model_validate_json(config_json)
    worker = InferenceWorker(idx)

    async def serve() -> None:
        try:
            await worker.initialize(cfg)
        except BaseException as e:  # noqa: BLE001 - the parent must hear about it
            if conn is not None:
                conn.send((0, None, "%s\n%s" % (e, traceback.format_exc())))
            raise
        if rank != 0:
            loop = asyncio.get_running_loop()
            await loop.run_in_executor(None, worker.run_follower)
            return
        conn.send((0, "ready", None))
        loop = asyncio.get_running_loop()
        pending = set()

        async def handle(cid, method, kwargs):
            try:
                res = await getattr(worker, method)(**kwargs)
                conn.send((cid, res, None))
            except BaseException as e:  # noqa: BLE001
                conn.send((cid, None, "%s: %s" % (type(e).__name__, e)))

        while True:
            msg = await loop.run_in_executor(None, conn.recv)
            if msg is None:
                break
            cid, method, kwargs = msg
            t = asyncio.ensure_future(handle(cid, method, kwargs))
            pending.add(t)
            t.add_done_callback(pending.discard)
            if method == "shutdown":
                await t
                break

    asyncio.run(serve())


class ProcessWorker(WorkerBase):
    """Same interface as :class:`InferenceWorker`, engine in child processes."""

    def __init__(self, idx: int = 0, gpu_ids: Optional[list] = None, master_port: int = 0,
                 start_timeout: float = 1800.0):
        super().__init__(idx)
        self.gpu_ids = gpu_ids
        self.master_port = master_port or (29600 + 7 * idx)
        self.start_timeout = start_timeout
        self.procs: list = []
        self.conn = None
        self._futs: dict[int, tuple] = {}
        self._cid = 0
        self._reader: Optional[threading.Thread] = None
        self._lock = threading.Lock()

    async def initialize(self, config) -> None:
        ctx = mp.get_context("spawn")
        world = config.world_size
        env = {k: str(v) for k, v in (config.extra_env or {}).items()}
        if self.gpu_ids is not None:
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(g) for g in self.gpu_ids)
        env.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(self.master_port), WORLD_SIZE=str(world))
        parent, child = ctx.Pipe()
        self.conn = parent
        for r in range(world):
            e = dict(env, RANK=str(r), LOCAL_RANK=str(r))
            p = ctx.Process(target=_child_main, daemon=True,
                            args=(child if r == 0 else None, self.idx, r, e, config.model_dump_json()))
            p.start()
            self.procs.append(p)
        loop = asyncio.get_running_loop()
        ok = await loop.run_in_executor(None, parent.poll, self.start_timeout)
        if not ok:
            await self.shutdown()
            raise TimeoutError("worker %d did not start within %.0f s" % (self.idx, self.start_timeout))
        _, res, err = parent.recv()
        if err is not None:
            await self.shutdown()
            raise RuntimeError("worker %d failed to start: %s" % (self.idx, err))
        self.config = config
        self.status = WorkerStatus.READY
        self._loop = loop
        self._reader = threading.Thread(target=self._read, name="worker-%d-reader" % self.idx,
                                        daemon=True)
        self._reader.start()

    def _read(self) -> None:
        try:
            while True:
                cid, res, err = self.conn.recv()
                ent = self._futs.pop(cid, None)
                if ent is None:
                    continue
                loop, fut = ent
                loop.call_soon_threadsafe(_settle, fut, res, err)
        except (EOFError, OSError):
            for cid, (loop, fut) in list(self._futs.items()):
                loop.call_soon_threadsafe(_settle, fut, None, "worker process exited")
            self._futs.clear()

    async def _rpc(self, method: str, **kwargs):
        if self.conn is None:
            raise ConnectionError("worker %d is not running" % self.idx)
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            self._cid += 1
            cid = self._cid
            self._futs[cid] = (loop, fut)
            try:
                self.conn.send((cid, method, kwargs))
            except (OSError, ValueError) as e:
                self._futs.pop(cid, None)
                raise ConnectionError("worker %d pipe closed: %s" % (self.idx, e))
        return await fut

    async def generate(self, prompt, sampling_params=None, request_id=None, routing_key=None) -> dict:
        return await self._rpc("generate", prompt=prompt, sampling_params=sampling_params,
                               request_id=request_id, routing_key=routing_key)

    async def cancel_inflight(self) -> int:
        return await self._rpc("cancel_inflight")

    async def get_stats(self) -> dict:
        return await self._rpc("get_stats")

    async def health(self) -> bool:
        if not self.procs or any(not p.is_alive() for p in self.procs):
            return False
        try:
            return bool(await asyncio.wait_for(self._rpc("health"), timeout=10))
        except Exception:  # noqa: BLE001
            return False

    async def sleep(self, level: int = 1) -> None:
        await self._rpc("sleep", level=level)
        self.status = WorkerStatus.SLEEPING

    async def wake_up(self, tags=None) -> None:
        await self._rpc("wake_up", tags=tags)
        done = not tags or "kv_cache" in tags
        self.status = WorkerStatus.READY if done else WorkerStatus.WEIGHTS_READY

    async def reset_prefix_cache(self) -> None:
        await self._rpc("reset_prefix_cache")

    async def weights_info(self) -> list[dict]:
        return await self._rpc("weights_info")

    async def spec_weights_info(self) -> list[dict]:
        return await self._rpc("spec_weights_info")

    async def sync_weights(self, **kw) -> dict:
        return await self._rpc("sync_weights", **kw)

    async def sync_spec_weights(self, **kw) -> dict:
        return await self._rpc("sync_spec_weights", **kw)

    async def close_weight_sync(self) -> dict:
        return await self._rpc("close_weight_sync")

    async def compute_weight_norm(self) -> float:
        return await self._rpc("compute_weight_norm")

    async def shutdown(self) -> None:
        if self.conn is not None and self.status is not WorkerStatus.UNINITIALIZED:
            try:
                await asyncio.wait_for(self._rpc("shutdown"), timeout=30)
            except Exception:  # noqa: BLE001
                pass
        for p in self.procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
        self.procs = []
        if self.conn is not None:
            self.conn.close()
            self.conn = None
        self.status = WorkerStatus.UNINITIALIZED


def _settle(fut, res, err) -> None:
    if fut.done():
        return
    if err is not None:
        fut.set_exception(RuntimeError(err))
    else:
        fut.set_result(res)
