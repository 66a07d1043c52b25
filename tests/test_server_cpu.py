"""Replica-pool server on CPU: routing, admission control, pool life cycle, multi-model
driver, pipeline and the REST API, with deterministic fake workers."""

import asyncio
import pickle
import random

import pytest
from fastapi.testclient import TestClient

from arcticinference_b200.server import api
from arcticinference_b200.server.config import (GPUType, ServerModelConfig, normalize_model_name)
from arcticinference_b200.server.metrics import (BoundedRing, ConcurrencyHistory, RequestRecord,
                                                 WorkerMetricsCollector, summarize)
from arcticinference_b200.server.multi_model import Driver
from arcticinference_b200.server.pipeline import Pipeline, TaskError
from arcticinference_b200.server.replica_pool import GpuAllocator, ReplicaPool
from arcticinference_b200.server.scheduler import (PendingRequest, Scheduler, WorkerSlot,
                                                   fixed_concurrency, least_loaded_routing,
                                                   prefix_affinity_routing, stable_hash,
                                                   strict_affinity_routing,
                                                   utilization_based_concurrency)
from arcticinference_b200.server.testing import DummyWorker, dummy_tokens
from arcticinference_b200.server.worker import WorkerStatus

CFG = ServerModelConfig(model="llama-tiny", max_model_len=256)


def run(coro):
    return asyncio.run(coro)


# ------------------------------------------------------------------------------ config / metrics
def test_config_translation_and_registry():
    c = ServerModelConfig(model="m", use_fca=True, spec_model="spec", kv_cache_dtype=None,
                          extra_engine_kwargs={"block_size": 32})
    kw = c.to_engine_kwargs()
    assert kw["forest_cascade_attn_configs"] == "{}" and kw["block_size"] == 32
    assert kw["speculative_config"]["model"] == "spec" and "use_fca" not in kw and "kv_cache_dtype" not in kw
    off = ServerModelConfig(model="m", use_fca=True, spec_model="s",
                            extra_env={"ARCTIC_INFERENCE_ENABLED": "0"}).to_engine_kwargs()
    assert "speculative_config" not in off and "forest_cascade_attn_configs" not in off
    assert normalize_model_name("meta-llama/Llama-3.1-8B-Instruct-FP8") == "Llama-3.1-8B-Instruct"
    r = ServerModelConfig.from_registry("org/Llama-3.3-70B-Instruct-FP8", GPUType.B200, 8192)
    assert r.ulysses_sequence_parallel_size == 8 and r.enable_shift_parallel and r.world_size == 8
    with pytest.raises(ValueError):
        ServerModelConfig.from_registry("unknown", GPUType.B200)


def test_metrics_primitives():
    ring = BoundedRing(3)
    for i in range(5):
        ring.append(i)
    assert ring.dropped == 2
    clone = pickle.loads(pickle.dumps(ring))
    assert clone.drain() == [2, 3, 4] and len(clone) == 0 and ring.drain() == [2, 3, 4]
    col = WorkerMetricsCollector(1, min_interval=1.0)
    assert col.observe({"running": 2, "kv_cache_usage": 0.5}, 8, 2, now=10.0) is not None
    assert col.observe({"running": 3}, 8, 3, now=10.5) is None          # throttled
    assert col.observe({"running": 3}, 8, 3, now=11.1) is not None
    assert [s["running"] for s in col.drain()] == [2, 3]
    h = ConcurrencyHistory()
    h.record([8, 8], now=1.0)
    h.record([8, 8], now=2.0)               # unchanged: not stored
    h.record([10, 8], now=3.0)
    assert h.at(0.5) is None and h.at(2.5) == [8, 8] and h.at(9) == [10, 8]
    assert len(h.drain()) == 2 and h.at(9) == [10, 8]
    recs = [RequestRecord(i, 0, 0.0, 0.1, 1.0 + i, 10, 5) for i in range(4)] + \
        [RequestRecord(9, 0, 0, 0, 1, error="x")]
    s = summarize(recs)
    assert s["count"] == 5 and s["errors"] == 1 and s["p50_latency"] == 3.0


# ------------------------------------------------------------------------------ routing
def _slots(loads, limit=10, avail=None):
    return [WorkerSlot(None, limit, active_requests=a, available=(avail[i] if avail else True))
            for i, a in enumerate(loads)]


def _req(h=None):
    return PendingRequest(1, "p", {}, None, prefix_hash=h)


def test_routing_functions():
    assert least_loaded_routing(_req(), _slots([5, 1, 3])) == 1
    assert least_loaded_routing(_req(), _slots([5, 1, 3], avail=[True, False, True])) == 2
    w = _slots([0, 0, 0, 0])
    assert prefix_affinity_routing(_req(6), w) == 2
    w[2].active_requests = 9                                      # above 85 % of 10: spill to the next
    assert prefix_affinity_routing(_req(6), w) == 3
    assert strict_affinity_routing(_req(6), w) == 2                # never spills
    for s in w:
        s.active_requests = 9
    w[1].active_requests = 8
    assert prefix_affinity_routing(_req(6), w) == 1                # all hot: least loaded
    assert prefix_affinity_routing(_req(None), w) == 1
    w[2].available = False
    assert strict_affinity_routing(_req(6), w) == [0, 1, 3][6 % 3]
    assert stable_hash("abc") == stable_hash("abc") and stable_hash([1, 2]) != stable_hash([2, 1])


def test_concurrency_controller():
    rng = random.Random(0)
    mk = lambda **kw: WorkerSlot(None, kw.pop("limit", 64), **kw)
    grow = mk(active_requests=64, latest_cache_utilization=0.5, running_reqs=60)
    idle = mk(active_requests=10, latest_cache_utilization=0.5, running_reqs=10)
    hot = mk(active_requests=64, latest_cache_utilization=0.97, running_reqs=64)
    queued = mk(active_requests=64, latest_cache_utilization=0.92, running_reqs=60, waiting_reqs=5)
    cold = mk(active_requests=100, limit=8)
    lims = [utilization_based_concurrency([grow, idle, hot, queued, cold], rng) for _ in range(50)]
    assert all(l[0] == 64 + 2 + 4 for l in lims)          # gap 0.4 -> +2 +4
    assert all(l[1] == 64 for l in lims)                  # not pressing against its limit
    assert {l[2] for l in lims} == {63, 64} and {l[3] for l in lims} == {63, 64}
    assert all(l[4] == 95 for l in lims)                  # no statistics yet: follow offered load
    assert fixed_concurrency(5)([grow, idle]) == [5, 5]


# ------------------------------------------------------------------------------ scheduler / pool
def test_scheduler_limits_retries_and_records():
    async def main():
        ws = [DummyWorker(0, latency=0.02), DummyWorker(1, latency=0.02, fail_after=0)]
        for w in ws:
            await w.initialize(CFG)
        s = Scheduler(ws, routing_fn=least_loaded_routing, concurrency_fn=fixed_concurrency(2))
        await s.poll_once()
        peak = 0

        async def watch():
            nonlocal peak
            while s.inflight:
                peak = max(peak, ws[0].active)
                await asyncio.sleep(0.001)
        outs, _ = await asyncio.gather(s.submit_batch([[i, i + 1] for i in range(8)], {"max_tokens": 4}),
                                       watch())
        assert [o["token_ids"] for o in outs] == [dummy_tokens([i, i + 1], 4) for i in range(8)]
        assert peak <= 2                                       # the admission limit held
        assert not s.workers[1].available                      # connection errors take a worker out
        m = s.drain_metrics()
        assert len(m["requests"]) == 8 and all(r["worker_idx"] == 0 for r in m["requests"])
        assert any(r["retries"] > 0 for r in m["requests"]) and s.drain_metrics()["requests"] == []
        s.pause()
        with pytest.raises(RuntimeError, match="paused"):
            await s.submit([1], {})
        with pytest.raises(ValueError):
            s.resume()
            await s.submit_batch([[1], [2]], {}, routing_key=["a"])
        await s.close()
    run(main())


def _pool(n=3, **kw):
    made = []

    def factory(i):
        w = DummyWorker(i, **kw)
        made.append(w)
        return w
    return ReplicaPool(worker_factory=factory, gpu_ids=list(range(8))), made


def test_pool_generate_affinity_sleep_scale():
    async def main():
        pool, made = _pool(3)
        assert await pool.initialize(CFG, model_id="m", num_replicas=3) == 3
        assert pool.allocator.free == [3, 4, 5, 6, 7]
        one = await pool.generate([1, 2, 3], {"max_tokens": 3})
        assert one[0]["token_ids"] == dummy_tokens([1, 2, 3], 3) and one[0]["prompt_len"] == 3
        # same routing key -> same replica, whatever the prompt
        await pool.generate([[i] * 3 for i in range(12)], {"max_tokens": 2}, routing_key="conv-7", strict=True)
        assert sorted(len(w.seen) for w in made)[:2] == [0, 0] or sum(len(w.seen) > 1 for w in made) == 1
        with pytest.raises(ValueError):
            await pool.generate([1, 2], {}, routing_key=["a", "b"])
        with pytest.raises(ValueError):
            await pool.generate("x", {}, model_id="other")
        # sleep -> staged wake
        assert (await pool.sleep("m", level=2))["status"] == "sleeping"
        with pytest.raises(RuntimeError, match="sleeping"):
            await pool.generate("x", {})
        assert (await pool.wake_up("m", tags=["weights"]))["status"] == "weights_ready"
        assert all(w.status is WorkerStatus.WEIGHTS_READY for w in made) and pool.sleeping
        assert (await pool.wake_up("m", tags=["kv_cache"]))["status"] == "awake"
        assert (await pool.generate("again", {"max_tokens": 1}))[0]["generation_len"] == 1
        # scaling
        await pool.scale_up(5)
        assert pool.num_replicas == 5 and pool.allocator.free == [5, 6, 7]
        await pool.scale_down(2)
        assert pool.num_replicas == 2 and pool.allocator.free == [2, 3, 4, 5, 6, 7]
        st = await pool.get_status()
        assert st["num_replicas"] == 2 and st["workers"][1]["gpus"] == [1]
        assert (await pool.reset_prefix_cache())["replicas"] == 2
        await pool.shutdown()
        assert pool.allocator.free == list(range(8)) and (await pool.get_status()) == {"initialized": False}
    run(main())


def test_pool_sync_strategies_and_health():
    async def main():
        pool, made = _pool(2, latency=0.05)
        await pool.initialize(CFG, num_replicas=2)
        groups = [{"group_id": 0, "master_addr": "127.0.0.1", "master_port": 5000, "world_size": 3,
                   "replica_ids": [0, 1]}]
        # hotswap: traffic keeps flowing
        gen = asyncio.ensure_future(pool.generate([[i] for i in range(6)], {"max_tokens": 2}))
        await asyncio.sleep(0.01)
        r = await pool.sync_weights(groups=groups, strategy="hotswap")
        assert r["replicas"] == [0, 1] and all(w.weights_version == 1 for w in made)
        assert len(await gen) == 6
        # drain: waits for in-flight work, refuses new work meanwhile
        gen = asyncio.ensure_future(pool.generate([[i] for i in range(4)], {"max_tokens": 2}))
        await asyncio.sleep(0.01)
        sync = asyncio.ensure_future(pool.sync_weights(master_addr="127.0.0.1", master_port=5000,
                                                       strategy="drain"))
        await asyncio.sleep(0.01)
        with pytest.raises(RuntimeError, match="paused"):
            await pool.generate([9], {})
        assert len(await gen) == 4 and (await sync)["strategy"] == "drain"
        assert (await pool.generate([9], {"max_tokens": 1}))[0]["generation_len"] == 1
        # skip: in-flight requests are cancelled and transparently retried
        gen = asyncio.ensure_future(pool.generate([[i, 7] for i in range(4)], {"max_tokens": 2}))
        await asyncio.sleep(0.01)
        await pool.sync_weights(groups=groups, strategy="skip")
        outs = await gen
        assert [o["token_ids"] for o in outs] == [dummy_tokens([i, 7], 2) for i in range(4)]
        assert all(w.weights_version == 3 for w in made)
        with pytest.raises(ValueError):
            await pool.sync_weights(groups=groups, strategy="nope")
        with pytest.raises(ValueError):
            await pool.sync_weights(strategy="drain")
        # health: a dead replica is replaced
        made[1].status = WorkerStatus.UNINITIALIZED
        assert await pool.check_health_once() == [1]
        assert pool.restarts == 1 and len(made) == 3 and made[2].status is WorkerStatus.READY
        assert (await pool.generate([[5], [6], [7], [8]], {"max_tokens": 1}))[3]["generation_len"] == 1
        await pool.shutdown()
    run(main())


def test_driver_shares_gpus_between_models():
    async def main():
        d = Driver(worker_factory=lambda i: DummyWorker(i), gpu_ids=list(range(8)))
        assert await d.initialize(CFG, model_id="a") == 8
        two = ServerModelConfig(model="llama-tiny", tensor_parallel_size=2)
        assert await d.initialize(two, model_id="b") == 2            # a shrinks to 4, b gets 4 GPUs
        st = await d.get_status()
        assert st["models"]["a"]["num_replicas"] == 4 and st["free_gpus"] == 0
        assert (await d.generate([1, 2], {"max_tokens": 2}, model_id="b"))[0]["generation_len"] == 2
        with pytest.raises(ValueError):
            await d.generate([1], {})                                # two models: id required
        with pytest.raises(KeyError):
            await d.generate([1], {}, model_id="zzz")
        await d.shutdown("b")
        await d.wait_scaling()
        assert (await d.get_status())["models"]["a"]["num_replicas"] == 8
        big = ServerModelConfig(model="llama-tiny", tensor_parallel_size=8)
        with pytest.raises(RuntimeError, match="not enough GPUs"):
            await d.initialize(big, model_id="c")
        await d.shutdown()
    run(main())


def test_pipeline_retries_and_order():
    async def main():
        pool, _ = _pool(2)
        await pool.initialize(CFG, num_replicas=2)
        pipe = Pipeline(pool)
        flaky = {"left": 3}

        @pipe.task(max_in_flight=4, retries=2)
        async def job(item, generate):
            if item["id"] % 5 == 0 and flaky["left"] > 0:
                flaky["left"] -= 1
                raise RuntimeError("transient")
            out = await generate(item["prompt"], {"max_tokens": 2})
            return item["id"], out["token_ids"]

        data = [{"id": i, "prompt": [i, i]} for i in range(12)]
        seen = []
        res = await job.run(data, progress=lambda a, b: seen.append((a, b)))
        assert [r[0] for r in res] == list(range(12)) and res[3][1] == dummy_tokens([3, 3], 2)
        assert seen[-1] == (12, 12) and job.attempts == 15

        @pipe.task(retries=1, return_exceptions=True)
        async def bad(item, generate):
            raise ValueError("always")
        out = await bad.run([1, 2])
        assert all(isinstance(o, TaskError) for o in out)

        @pipe.task(retries=0)
        async def fatal(item, generate):
            raise ValueError("boom")
        with pytest.raises(TaskError):
            await fatal.run([1])
        await pool.shutdown()
    run(main())


def test_pipeline_in_the_reference_call_shape():
    """``@pipeline.task`` + ``await pipeline.run(dataset)`` with an LLM handle whose
    ``generate`` / ``generate_token_ids`` take sampling parameters as keywords."""
    async def main():
        pool, _ = _pool(2)
        await pool.initialize(CFG, num_replicas=2)
        pipe = Pipeline(pool)
        pipe.retry_delay = 0.01
        with pytest.raises(RuntimeError, match="no task"):
            await pipe.run([1])
        with pytest.raises(ValueError, match="async"):
            pipe.task(lambda sample, llm: None)
        flaky = {"left": 2}

        @pipe.task
        async def process(sample, llm):
            if sample["id"] == 1 and flaky["left"] > 0:
                flaky["left"] -= 1
                raise RuntimeError("transient")
            if sample["id"] == 4:
                raise ValueError("never works")
            ids = await llm.generate_token_ids(sample["ids"], max_tokens=3)
            text = await llm.generate(prompt=sample["ids"], max_tokens=3)
            return {"id": sample["id"], "ids": ids, "text": text}

        data = [{"id": i, "ids": [i, i + 1]} for i in range(6)]
        res = await pipe.run(data, max_retries=2, show_progress=False)
        assert [r.get("id") for r in res] == [0, 1, 2, 3, None, 5]
        assert res[4] == {"__error__": "never works"}
        assert res[2]["ids"] == dummy_tokens([2, 3], 3) and isinstance(res[2]["text"], str)

        # several pools: the task gets a dict of handles
        both = Pipeline({"a": pool, "b": pool})

        @both.task
        async def two(sample, llms):
            return [await llms[k].generate_token_ids(sample, max_tokens=1) for k in ("a", "b")]
        out = await both.run([[7, 8]], max_retries=0)
        assert out[0][0] == out[0][1] == dummy_tokens([7, 8], 1)
        await pool.shutdown()
    run(main())


def test_rest_api():
    pool, made = _pool(2)
    api.set_backend(pool)
    with TestClient(api.app) as c:
        assert c.get("/status").json() == {"initialized": False}
        r = c.post("/init", json={"config": {"model": "llama-tiny"}, "model_id": "m", "num_replicas": 2})
        assert r.status_code == 200 and r.json()["num_replicas"] == 2
        r = c.post("/generate", json={"prompts": [[1, 2], "some text"], "sampling_params": {"max_tokens": 3}})
        assert [x["generation_len"] for x in r.json()["results"]] == [3, 3]
        assert c.get("/weights_info").json()["count"] == 1
        g = {"group_id": 0, "master_addr": "127.0.0.1", "master_port": 5000, "world_size": 3, "replica_ids": [0, 1]}
        assert c.post("/sync_weights", json={"groups": [g], "strategy": "drain"}).json()["status"] == "ok"
        assert c.post("/sync_weights", json={"strategy": "bogus", "groups": [g]}).status_code == 500
        assert c.post("/sleep", json={"model_id": "m", "level": 1}).json()["status"] == "sleeping"
        assert c.post("/generate", json={"prompts": ["x"]}).status_code == 503
        assert c.post("/wake_up", json={"model_id": "m"}).json()["status"] == "awake"
        m = c.get("/metrics").json()
        assert len(m["requests"]) == 2 and c.get("/metrics").json()["requests"] == []
        assert c.post("/reset_prefix_cache").status_code == 200
        assert c.post("/close_weight_sync").json()["status"] == "ok"
        assert c.post("/shutdown").json()["status"] == "shutdown"
    api.set_backend(ReplicaPool())


def test_gpu_allocator():
    a = GpuAllocator([4, 5, 6])
    assert a.acquire(2) == [4, 5]
    with pytest.raises(RuntimeError):
        a.acquire(2)
    a.release([4, 5])
    assert a.free == [4, 5, 6] and GpuAllocator([]).acquire(4) is None


def test_process_worker_hosts_engine_in_child():
    from arcticinference_b200.server.worker import ProcessWorker

    async def main():
        w = ProcessWorker(0, gpu_ids=None, master_port=29877, start_timeout=300)
        cfg = ServerModelConfig(model="llama-tiny", max_model_len=128, max_num_seqs=8,
                                extra_env={"CUDA_VISIBLE_DEVICES": ""},
                                extra_engine_kwargs={"num_gpu_blocks_override": 64, "block_size": 16})
        await w.initialize(cfg)
        try:
            assert await w.health()
            sp = {"temperature": 0.0, "max_tokens": 5, "ignore_eos": True}
            a, b = await asyncio.gather(w.generate([1, 2, 3], sp), w.generate([1, 2, 3], sp))
            assert a["token_ids"] == b["token_ids"] and a["generation_len"] == 5 and a["prompt_len"] == 3
            st = await w.get_stats()
            assert st["generation_tokens"] >= 10
            assert len(await w.weights_info()) == 21
            with pytest.raises(RuntimeError):
                await w.generate([1], {"temperature": -3})
            await w.sleep(1)
            assert w.status is WorkerStatus.SLEEPING
            await w.wake_up()
            assert (await w.generate([4, 5], sp))["generation_len"] == 5
        finally:
            await w.shutdown()
        assert not await w.health()
    run(main())
