"""Embedding path on CPU: encoder numerics against an independent PyTorch restatement,
batch planning, the asynchronous engine, wire messages and the gRPC replica / manager /
client chain (all in one process, tiny random model)."""

import asyncio
import math

import numpy as np
import pytest
import torch

from arcticinference_b200.config import ModelConfig
from arcticinference_b200.embedding import messages as pb
from arcticinference_b200.embedding.client import EmbeddingError, InferenceClient
from arcticinference_b200.embedding.engine import AsyncEmbeddingEngine, EmbeddingEngine
from arcticinference_b200.embedding.replica import InferenceServer, InferenceServicer
from arcticinference_b200.embedding.replica_manager import (ManagerServicer, ReplicaInfo,
                                                            ReplicaManager)
from arcticinference_b200.models.bert import BertEncoder, random_bert_state


def _torch_bert(cfg, state, ids, pooling="cls"):
    """Plain fp32 BERT forward of one sequence from HF-named weights."""
    w = {k: v.float() for k, v in state.items()}
    H, nh = cfg.hidden_size, cfg.num_attention_heads
    n = len(ids)
    x = w["embeddings.word_embeddings.weight"][ids] + \
        w["embeddings.position_embeddings.weight"][:n] + w["embeddings.token_type_embeddings.weight"][0]
    ln = lambda t, p: torch.nn.functional.layer_norm(t, (H,), w[p + ".weight"], w[p + ".bias"],
                                                     cfg.layer_norm_eps)
    x = ln(x, "embeddings.LayerNorm")
    for l in range(cfg.num_hidden_layers):
        p = "encoder.layer.%d." % l
        lin = lambda t, q: t @ w[p + q + ".weight"].t() + w[p + q + ".bias"]
        q, k, v = (lin(x, "attention.self." + s).view(n, nh, -1).transpose(0, 1)
                   for s in ("query", "key", "value"))
        a = torch.softmax(q @ k.transpose(1, 2) / math.sqrt(q.shape[-1]), -1) @ v
        a = a.transpose(0, 1).reshape(n, H)
        x = ln(x + lin(a, "attention.output.dense"), p + "attention.output.LayerNorm")
        u = torch.nn.functional.gelu(lin(x, "intermediate.dense"))
        x = ln(x + lin(u, "output.dense"), p + "output.LayerNorm")
    v = x[0] if pooling == "cls" else x.mean(0)
    return v / v.norm()


@pytest.fixture(scope="module")
def tiny_engine():
    return EmbeddingEngine("bert-tiny", device="cpu", dtype=torch.float32,
                           max_num_batched_tokens=512, max_num_seqs=8)


@pytest.mark.parametrize("pooling", ["cls", "mean"])
def test_encoder_matches_plain_torch(tiny_engine, pooling):
    cfg = tiny_engine.cfg
    state = dict(random_bert_state(cfg, 0, 0.02, "cpu", torch.float32))
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (5, 17, 1, 64)]
    got = tiny_engine.encode(seqs, pooling=pooling)
    for s, g in zip(seqs, got):
        want = _torch_bert(cfg, state, torch.tensor(s), pooling)
        assert np.allclose(g, want.numpy(), atol=2e-5), float(np.abs(g - want.numpy()).max())


def test_fused_qkv_loading_accepts_bert_prefix():
    cfg = ModelConfig.from_pretrained("bert-tiny")
    enc = BertEncoder(cfg, "cpu", torch.float32)
    enc.load_state(("bert." + k, v) for k, v in random_bert_state(cfg, 3, 0.02, "cpu", torch.float32))
    assert enc.layers[0].wqkv.shape == (3 * cfg.hidden_size, cfg.hidden_size)
    assert enc.num_parameters() > 0
    with pytest.raises(ValueError):
        BertEncoder(cfg, "cpu", torch.float32).load_state([])


def test_batch_planning_respects_budgets(tiny_engine):
    lens = [512, 300, 200, 100, 50, 50, 10, 5, 1, 1, 1, 1]
    batches = tiny_engine.plan_batches(lens)
    assert sorted(i for b in batches for i in b) == list(range(len(lens)))
    for b in batches:
        assert len(b) <= tiny_engine.max_seqs
        assert sum(lens[i] for i in b) <= tiny_engine.max_tokens
    # many batches, results land in request order; over-long input is truncated
    rng = np.random.default_rng(1)
    seqs = [rng.integers(0, 1000, size=n).tolist() for n in [400, 3, 600, 200, 7, 9, 300, 2, 2, 2, 2]]
    all_at_once = tiny_engine.encode(seqs)
    one_by_one = np.stack([tiny_engine.encode([s])[0] for s in seqs])
    assert np.allclose(all_at_once, one_by_one, atol=1e-5)
    assert np.allclose(tiny_engine.encode([seqs[2][:512]])[0], all_at_once[2], atol=1e-5)


def test_async_engine_merges_and_aborts(tiny_engine):
    async def run():
        a = AsyncEmbeddingEngine(tiny_engine, max_wait_ms=20)
        try:
            before = tiny_engine.stats.batches
            outs = await asyncio.gather(*[a.encode([[i + 1, i + 2, i + 3]], request_id="r%d" % i)
                                          for i in range(6)])
            assert tiny_engine.stats.batches - before < 6       # merged into fewer batches
            for i, o in enumerate(outs):
                assert np.allclose(o, tiny_engine.encode([[i + 1, i + 2, i + 3]]), atol=1e-6)
            assert a.abort("unknown") is False
        finally:
            a.stop()
    asyncio.run(run())


def test_wire_messages_roundtrip():
    ids = np.array([101, 7, 102], dtype="<i4")
    r = pb.EncodeRequest(request_id="x", n_prompts=1, token_id_bytes_i32=[ids.tobytes()], priority=2)
    back = pb.EncodeRequest.FromString(r.SerializeToString())
    assert np.frombuffer(back.token_id_bytes_i32[0], "<i4").tolist() == [101, 7, 102]
    # field numbers are the published ones: tag of field 4, wire type 2 = 0x22
    assert b"\x22\x0c" in r.SerializeToString()
    assert pb.method_path("Encode") == "/arctic_inference.InferenceService/Encode"


def test_grpc_replica_manager_client(tiny_engine):
    async def run():
        servers, infos = [], []
        for _ in range(2):
            s = InferenceServer(InferenceServicer(tiny_engine, "bert-tiny"), "127.0.0.1", 0)
            port = await s.start()
            servers.append(s)
            infos.append(ReplicaInfo("127.0.0.1", port))
        mgr = ReplicaManager(infos, load_balancing="round_robin", health_interval=0.2)
        await mgr.start()
        front = InferenceServer(ManagerServicer(mgr), "127.0.0.1", 0)
        fport = await front.start()
        try:
            async with InferenceClient("127.0.0.1", fport) as c:
                assert await c.health_check()
                info = await c.get_replica_info()
                assert info["n_replicas"] == 2 and info["n_healthy_replicas"] == 2
                assert info["replicas"][0]["task"] == "embed"
                toks = [[5, 6, 7], [9] * 40]
                v = await c.embed(token_ids=toks)
                assert v.shape == (2, tiny_engine.cfg.hidden_size)
                assert np.allclose(v, tiny_engine.encode(toks), atol=1e-6)
                assert np.allclose(np.linalg.norm(v, axis=1), 1.0, atol=1e-4)
                t = await c.embed(prompts=["hello world"])
                assert t.shape[0] == 1
                for _ in range(4):
                    await c.embed(token_ids=[[1, 2]])
                assert all(r.served >= 2 for r in mgr.replicas)          # both were used
                with pytest.raises(EmbeddingError):
                    await c.embed(token_ids=[[1]], model_name="other-model")
                assert (await c.abort("nothing"))["success"] is False
                # one replica goes away: requests keep flowing through the other
                await servers[0].server.stop(0)
                for _ in range(3):
                    assert (await c.embed(token_ids=[[3, 4]])).shape[0] == 1
                await asyncio.sleep(0.5)
                assert (await c.get_replica_info())["n_healthy_replicas"] == 1
        finally:
            await front.server.stop(0)
            await mgr.stop()
            for s in servers[1:]:
                await s.server.stop(0)
    asyncio.run(run())


def test_least_loaded_and_random_policies():
    reps = [ReplicaInfo("h", 1, healthy=True, inflight=3), ReplicaInfo("h", 2, healthy=True, inflight=1),
            ReplicaInfo("h", 3, healthy=False, inflight=0)]
    assert ReplicaManager(reps, "least_loaded").select_replica().port == 2
    assert ReplicaManager(reps, "random").select_replica().port in (1, 2)
    assert ReplicaManager([reps[2]], "round_robin").select_replica() is None


def test_manager_launches_replica_processes():
    async def run():
        mgr = ReplicaManager(load_balancing="least_loaded", health_interval=0.5, startup_timeout=240)
        try:
            await mgr.launch("bert-tiny", 2, base_port=18510, host="127.0.0.1", devices=["cpu", "cpu"],
                             extra=["--max-num-batched-tokens", "1024"])
            assert [r.healthy for r in mgr.replicas] == [True, True]
            assert mgr.replicas[0].port != mgr.replicas[1].port
            front = InferenceServer(ManagerServicer(mgr), "127.0.0.1", 0)
            port = await front.start()
            async with InferenceClient("127.0.0.1", port) as c:
                v = await c.embed(token_ids=[[1, 2, 3], [4, 5]])
                assert v.shape == (2, 128)
                assert (await c.get_replica_info())["n_healthy_replicas"] == 2
                # a replica process dies: the manager notices and keeps serving from the other
                mgr.replicas[0].process.terminate()
                mgr.replicas[0].process.wait(timeout=20)
                for _ in range(4):
                    assert (await c.embed(token_ids=[[7, 8, 9]])).shape == (1, 128)
                await asyncio.sleep(1.0)
                assert (await c.get_replica_info())["n_healthy_replicas"] == 1
            await front.server.stop(0)
        finally:
            await mgr.stop()
    asyncio.run(run())


def test_openai_embeddings_endpoint(tiny_engine):
    """/v1/embeddings: the four input shapes, both encodings, shortened vectors, errors."""
    import base64
    from fastapi.testclient import TestClient
    from arcticinference_b200.embedding.engine import AsyncEmbeddingEngine
    from arcticinference_b200.embedding.http_server import build_app, normalise_input

    assert normalise_input("a b") == ["a b"]
    assert normalise_input([1, 2, 3]) == [[1, 2, 3]]
    with pytest.raises(ValueError):
        normalise_input([[1], "x"])
    aeng = AsyncEmbeddingEngine(tiny_engine, max_wait_ms=0.5)
    try:
        with TestClient(build_app(aeng, "bert-tiny")) as c:
            ids = [[5, 6, 7, 8], [9, 10]]
            exp = tiny_engine.encode(ids)
            r = c.post("/v1/embeddings", json={"model": "bert-tiny", "input": ids})
            assert r.status_code == 200
            body = r.json()
            assert body["usage"]["prompt_tokens"] == 6 and len(body["data"]) == 2
            got = np.array([d["embedding"] for d in body["data"]], dtype=np.float32)
            np.testing.assert_allclose(got, exp, atol=1e-5)
            r = c.post("/v1/embeddings", json={"input": ids[0], "encoding_format": "base64"})
            v = np.frombuffer(base64.b64decode(r.json()["data"][0]["embedding"]), dtype="<f4")
            np.testing.assert_allclose(v, exp[0], atol=1e-5)
            r = c.post("/v1/embeddings", json={"input": ["hello world", "x"], "dimensions": 8})
            short = np.array([d["embedding"] for d in r.json()["data"]])
            assert short.shape == (2, 8)
            np.testing.assert_allclose(np.linalg.norm(short, axis=1), 1.0, atol=1e-5)
            assert c.post("/v1/embeddings", json={"input": []}).status_code == 400
            assert c.post("/v1/embeddings", json={"input": "x", "encoding_format": "hex"}).status_code == 400
            assert c.get("/v1/models").json()["data"][0]["id"] == "bert-tiny"
            assert c.get("/stats").json()["sequences"] >= 5
    finally:
        aeng.stop()


def test_replica_metrics_endpoint(tiny_engine):
    import socket
    import urllib.request
    from arcticinference_b200.embedding.replica import start_metrics_server
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server, thread = start_metrics_server(tiny_engine, port, "127.0.0.1")
    try:
        before = tiny_engine.stats.sequences
        tiny_engine.encode([[5, 6, 7], [8, 9]])
        text = urllib.request.urlopen("http://127.0.0.1:%d/metrics" % port, timeout=10).read().decode()
        assert "ab200_embedding_sequences_total %.1f" % (before + 2) in text
        assert "ab200_embedding_tokens_total" in text and "ab200_embedding_busy_seconds" in text
    finally:
        server.shutdown()
        thread.join(5)
