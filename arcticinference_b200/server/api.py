"""REST front end of the replica pool.

Endpoints and request bodies are those of the reference (arctic_inference/server/api.py:18-213):
``POST /init /generate /sleep /wake_up /sync_weights /sync_spec_weights /close_weight_sync
/shutdown`` and ``GET /weights_info /spec_weights_info /status /metrics``. ``/generate`` answers
503 while the pool is paused (draining for a weight update) or when the request was cancelled
by one, so that clients retry. ``backend`` is a :class:`ReplicaPool`; ``use_driver()`` swaps in
the multi-model :class:`Driver`.
"""

from __future__ import annotations

from contextlib import asynccontextmanager
from typing import Any, Optional, Union

from fastapi import FastAPI, HTTPException
from pydantic import BaseModel, Field

from .config import ServerModelConfig
from .replica_pool import ReplicaPool


class InitRequest(BaseModel):
    config: ServerModelConfig
    model_id: Optional[str] = None
    num_replicas: Optional[int] = None


class GenerateRequest(BaseModel):
    model_id: Optional[str] = None
    prompts: list[Union[str, list[int]]]
    sampling_params: dict[str, Any] = Field(default_factory=dict)
    routing_key: Union[str, list[Optional[str]], None] = None
    strict: bool = False


class GroupConfig(BaseModel):
    group_id: int
    master_addr: str
    master_port: int
    world_size: int
    replica_ids: list[int]


class SleepRequest(BaseModel):
    model_id: Optional[str] = None
    level: int = 1


class WakeUpRequest(BaseModel):
    model_id: Optional[str] = None
    tags: Optional[list[str]] = None


class SyncWeightsRequest(BaseModel):
    model_id: Optional[str] = None
    groups: Optional[list[GroupConfig]] = None
    bucket_size: int = 256 * 1024 * 1024
    strategy: str = "hotswap"
    engine_only: bool = False
    direct_mode: bool = False
    reverse: bool = False
    master_addr: Optional[str] = None
    master_port: Optional[int] = None
    world_size: Optional[int] = None


class SyncSpecWeightsRequest(BaseModel):
    model_id: Optional[str] = None
    groups: Optional[list[GroupConfig]] = None
    bucket_size: int = 256 * 1024 * 1024
    strategy: str = "hotswap"
    engine_only: bool = False
    reverse: bool = False
    master_addr: Optional[str] = None
    master_port: Optional[int] = None
    world_size: Optional[int] = None


backend: Any = ReplicaPool()


def set_backend(b: Any) -> None:
    global backend
    backend = b


def use_driver(**kw) -> Any:
    from .multi_model import Driver
    set_backend(Driver(**kw))
    return backend


@asynccontextmanager
async def lifespan(_app: FastAPI):
    yield
    await backend.shutdown()


app = FastAPI(title="arcticinference_b200 replica server", lifespan=lifespan)


def _fail(e: Exception, code: int = 500):
    raise HTTPException(status_code=code, detail="%s: %s" % (type(e).__name__, e))


@app.post("/init")
async def init_endpoint(request: InitRequest):
    try:
        n = await backend.initialize(request.config, model_id=request.model_id,
                                     num_replicas=request.num_replicas)
        return {"status": "ready", "model_id": request.model_id, "num_replicas": n}
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/generate")
async def generate_endpoint(request: GenerateRequest):
    try:
        return {"results": await backend.generate(**request.model_dump())}
    except RuntimeError as e:
        msg = str(e).lower()
        _fail(e, 503 if ("paused" in msg or "cancelled" in msg or "sleeping" in msg) else 500)
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/sleep")
async def sleep_endpoint(request: SleepRequest):
    try:
        return await backend.sleep(request.model_id, level=request.level)
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/wake_up")
async def wake_up_endpoint(request: WakeUpRequest):
    try:
        return await backend.wake_up(request.model_id, tags=request.tags)
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/reset_prefix_cache")
async def reset_prefix_cache_endpoint(model_id: Optional[str] = None):
    try:
        return await backend.reset_prefix_cache(model_id)
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.get("/weights_info")
async def weights_info_endpoint(model_id: Optional[str] = None):
    try:
        infos = await backend.get_weights_info_async(model_id=model_id)
        return {"weights_info": infos, "count": len(infos)}
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/sync_weights")
async def sync_weights_endpoint(request: SyncWeightsRequest):
    try:
        return await backend.sync_weights(**request.model_dump())
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.get("/spec_weights_info")
async def spec_weights_info_endpoint(model_id: Optional[str] = None):
    try:
        infos = await backend.get_spec_weights_info_async(model_id=model_id)
        return {"weights_info": infos, "count": len(infos)}
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/sync_spec_weights")
async def sync_spec_weights_endpoint(request: SyncSpecWeightsRequest):
    try:
        return await backend.sync_spec_weights(**request.model_dump())
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/close_weight_sync")
async def close_weight_sync_endpoint(model_id: Optional[str] = None):
    try:
        return await backend.close_weight_sync(model_id=model_id)
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.get("/status")
async def status_endpoint():
    try:
        return await backend.get_status()
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.get("/metrics")
async def metrics_endpoint(model_id: Optional[str] = None):
    """Everything recorded since the previous call (the server-side rings are emptied)."""
    try:
        return await backend.drain_metrics(model_id=model_id)
    except Exception as e:  # noqa: BLE001
        _fail(e)


@app.post("/shutdown")
async def shutdown_endpoint(model_id: Optional[str] = None):
    try:
        await backend.shutdown(model_id=model_id)
        return {"status": "shutdown", "model_id": model_id}
    except Exception as e:  # noqa: BLE001
        _fail(e)
