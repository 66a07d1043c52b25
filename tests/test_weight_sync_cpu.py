"""Weight synchronisation on CPU: transfer plan, the two-party channel (gloo), in-place
update of a live engine (bf16 and fp8, plain and SwiftKV), the reverse direction, the
shared-memory hand-over, and the full path through worker and pool."""

import asyncio
import os
import threading

import pytest
import torch

from arcticinference_b200.config import EngineArgs, ModelConfig
from arcticinference_b200.engine.llm_engine import LLMEngine
from arcticinference_b200.engine.sampling_params import SamplingParams
from arcticinference_b200.models.loader import random_llama_state
from arcticinference_b200.server.config import ServerModelConfig
from arcticinference_b200.server.replica_pool import ReplicaPool
from arcticinference_b200.server.weight_sync import TensorMeta, TransferSchedule, WeightSender
from arcticinference_b200.server.weight_sync.engine import Channel, ack, receive_stream, send_stream
from arcticinference_b200.server.weight_sync.ipc_engine import publish_ipc, wait_ipc_done
from arcticinference_b200.server.weight_sync.receiver import (engine_sync_weights,
                                                               engine_weights_info)
from arcticinference_b200.server.weight_sync.schedule import find_aliases
from arcticinference_b200.server.weight_sync.utils import (engine_weight_norm, export_llama_state)
from arcticinference_b200.server.worker import InferenceWorker

PORT = [41200]


def port(span: int = 8):
    """A base port with ``span`` consecutive free ports above it (a transfer to replica r, rank
    t listens on base + r * ranks + t). Probed by binding, because a fixed number can collide
    with an ephemeral port some other connection of the machine holds."""
    import socket
    base = PORT[0]
    while True:
        base += span
        if base + span >= 60000:
            base = 20000
        socks = []
        try:
            for p in range(base, base + span):
                sk = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
                socks.append(sk)
                sk.bind(("127.0.0.1", p))
            PORT[0] = base
            return base
        except OSError:
            continue
        finally:
            for sk in socks:
                sk.close()


def engine(model="llama-tiny", **kw):
    args = EngineArgs(model=model, num_gpu_blocks_override=64, block_size=16, max_model_len=128, **kw)
    return LLMEngine.from_engine_args(args, device="cpu")


def new_state(model="llama-tiny", seed=123):
    cfg = ModelConfig.from_pretrained(model)
    return dict(random_llama_state(cfg, seed, 0.05, "cpu", torch.bfloat16))


def greedy(eng, prompt=(3, 1, 4, 1, 5, 9, 2, 6)):
    eng.add_request("g", list(prompt), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    out = None
    while eng.has_unfinished_requests():
        for o in eng.step():
            out = o
    return out.outputs[0].token_ids


def test_schedule_packing():
    metas = [TensorMeta("model.layers.1.a", (100,), "bfloat16"), TensorMeta("model.layers.0.b", (300,), "float32"),
             TensorMeta("model.embed_tokens.weight", (64, 8), "bfloat16", direct=True),
             TensorMeta("model.layers.0.a", (1000,), "bfloat16"), TensorMeta("model.norm.weight", (8,), "bfloat16"),
             TensorMeta("lm_head.weight", (64, 8), "bfloat16", alias_of="model.embed_tokens.weight")]
    s = TransferSchedule.build(metas, bucket_size=2304)
    assert [m.name for m in s.direct] == ["model.embed_tokens.weight"] and len(s.aliases) == 1
    names = [[x.meta.name for x in b.slots] for b in s.buckets]
    assert names == [["model.norm.weight", "model.layers.0.a"], ["model.layers.0.b", "model.layers.1.a"]]
    for b in s.buckets:
        assert all(x.offset % 256 == 0 for x in b.slots) and b.nbytes <= 2304
    assert s.num_tensors == 5 and s.total_bytes == 16 + 2000 + 1200 + 200 + 1024
    big = TransferSchedule.build([TensorMeta("x", (10000,), "float32")], bucket_size=1024)
    assert len(big.buckets) == 1 and big.buckets[0].nbytes >= 40000
    a = torch.zeros(4)
    assert find_aliases({"p": a, "q": a, "r": torch.zeros(4)}) == {"q": "p"}


def test_channel_stream_roundtrip():
    p = port()
    g = torch.Generator().manual_seed(0)
    src = {"model.layers.%d.w" % i: torch.randn(37 + i, 5, generator=g).to(torch.bfloat16) for i in range(7)}
    src["model.embed_tokens.weight"] = torch.randn(50, 8, generator=g)
    src["lm_head.weight"] = src["model.embed_tokens.weight"]
    sender = WeightSender(src, device="cpu", direct_names=["model.embed_tokens.weight"])
    th = sender.start([{"master_addr": "127.0.0.1", "master_port": p, "replica_ids": [0]}],
                      bucket_size=1024, timeout=30)
    ch = Channel("127.0.0.1", p, rank=1, timeout=30)
    pre = torch.zeros(50, 8)
    got = {}
    for name, t in receive_stream(ch, lambda m: pre if m.name.startswith("model.embed") else None):
        got[name] = t if isinstance(t, str) else t.clone()
    ack(ch, len(got))
    stats = sender.join(th)
    assert stats[0]["applied"] == len(src) and got["lm_head.weight"] == "model.embed_tokens.weight"
    assert got["model.embed_tokens.weight"].data_ptr() != 0 and torch.equal(pre, src["model.embed_tokens.weight"])
    for k, v in src.items():
        if k != "lm_head.weight":
            assert torch.equal(got[k], v), k


@pytest.mark.parametrize("model,quant", [("llama-tiny", None), ("llama-tiny-swiftkv", None),
                                          ("llama-tiny", "fp8"), ("qwen3-tiny", None),
                                          ("qwen3-tiny", "fp8"), ("qwen2-tiny", None),
                                          ("qwen2-tiny", "fp8")])
def test_engine_update_matches_fresh_engine(model, quant):
    kw = {"quantization": quant} if quant else {}
    eng = engine(model, **kw)
    before = greedy(eng)
    ptr = eng.runner.model.layers[0].wo
    ptr = ptr.data_ptr() if isinstance(ptr, torch.Tensor) else ptr.q.data_ptr()
    state = new_state(model)
    p = port()
    sender = WeightSender(state, device="cpu", direct_names=["model.embed_tokens.weight", "lm_head.weight"])
    th = sender.start([{"master_addr": "127.0.0.1", "master_port": p, "replica_ids": [0]}],
                      bucket_size=1 << 20, timeout=60)
    res = engine_sync_weights(eng, {"master_addr": "127.0.0.1", "master_port": p, "timeout": 60})
    sender.join(th)
    assert res["incomplete_layers"] == [] and res["layers"] == eng.config.model.num_hidden_layers
    now = eng.runner.model.layers[0].wo
    assert (now.data_ptr() if isinstance(now, torch.Tensor) else now.q.data_ptr()) == ptr   # in place
    # oracle: an engine built from the same tensors through the checkpoint loader
    ref = engine(model, **kw)
    from arcticinference_b200.models.loader import load_llama_state
    load_llama_state(ref.runner.model, state.items())
    if quant:
        from arcticinference_b200.models.quant import quantize_model_fp8
        quantize_model_fp8(ref.runner.model)
    after, want = greedy(eng), greedy(ref)
    assert after == want and after != before
    assert abs(engine_weight_norm(eng) - engine_weight_norm(ref)) < 1e-3 * engine_weight_norm(ref)


def test_reverse_and_info():
    eng = engine()
    info = engine_weights_info(eng)
    names = {i["name"] for i in info}
    exported = dict(export_llama_state(eng.runner.model))
    assert names == set(exported) and all(tuple(exported[i["name"]].shape) == tuple(i["shape"]) for i in info)
    p = port()
    sender = WeightSender({"dummy": torch.zeros(1)}, device="cpu")
    th = sender.start([{"master_addr": "127.0.0.1", "master_port": p, "replica_ids": [0]}], reverse=True,
                      timeout=60)
    res = engine_sync_weights(eng, {"master_addr": "127.0.0.1", "master_port": p, "reverse": True,
                                    "bucket_size": 1 << 18})
    got = sender.join(th)[0]["received"]
    assert res["direction"] == "out" and set(got) == names
    assert all(torch.equal(got[k], exported[k]) for k in names)
    # what came out goes back in unchanged
    fresh = engine()
    from arcticinference_b200.models.loader import load_llama_state
    load_llama_state(fresh.runner.model, got.items())
    assert greedy(fresh) == greedy(eng)


def test_ipc_handover(tmp_path):
    eng = engine()
    state = new_state(seed=7)
    publish_ipc(state, "t1", shm_dir=str(tmp_path))
    res = {}
    th = threading.Thread(target=lambda: res.update(wait_ipc_done("t1", 60, shm_dir=str(tmp_path))))
    th.start()
    from arcticinference_b200.server.weight_sync.ipc_engine import receive_ipc
    r = receive_ipc(eng, "t1", shm_dir=str(tmp_path))
    th.join()
    assert r["transport"] == "ipc" and res["tensors"] == len(state)
    ref = engine()
    from arcticinference_b200.models.loader import load_llama_state
    load_llama_state(ref.runner.model, state.items())
    assert greedy(eng) == greedy(ref)


def test_pool_sync_with_real_workers():
    async def main():
        pool = ReplicaPool(worker_factory=lambda i: InferenceWorker(i, device="cpu"), gpu_ids=[])
        cfg = ServerModelConfig(model="llama-tiny", max_model_len=128, max_num_seqs=16,
                                extra_engine_kwargs={"num_gpu_blocks_override": 64, "block_size": 16})
        await pool.initialize(cfg, num_replicas=2)
        sp = {"temperature": 0.0, "max_tokens": 6, "ignore_eos": True}
        before = await pool.generate([[5, 6, 7, 8]] * 2, sp)
        info = await pool.get_weights_info_async()
        assert len(info) == 3 + 9 * 2
        state = new_state(seed=99)
        p = port() + 10
        groups = [{"group_id": 0, "master_addr": "127.0.0.1", "master_port": p, "world_size": 3,
                   "replica_ids": [0, 1]}]
        sender = WeightSender(state, device="cpu", direct_names=[i["name"] for i in info if i["direct"]])
        th = sender.start(groups, timeout=60)
        res = await pool.sync_weights(groups=groups, strategy="drain")
        await asyncio.get_running_loop().run_in_executor(None, sender.join, th)
        assert res["status"] == "ok" and [r["tensors"] for r in res["results"]] == [len(state)] * 2
        after = await pool.generate([[5, 6, 7, 8]] * 2, sp)
        assert after[0]["token_ids"] == after[1]["token_ids"] != before[0]["token_ids"]
        norms = (await pool.compute_weight_norm())["norms"]
        assert abs(norms[0] - norms[1]) < 1e-6
        assert (await pool.close_weight_sync())["status"] == "ok"
        await pool.shutdown()
    asyncio.run(main())


def test_transfer_plan_travels_as_validated_json():
    import json
    import pytest
    import torch
    from arcticinference_b200.server.weight_sync.schedule import TensorMeta, TransferSchedule
    metas = [TensorMeta.of("model.layers.%d.w" % i, torch.empty(64, 48, dtype=torch.bfloat16))
             for i in range(5)]
    metas.append(TensorMeta.of("model.embed", torch.empty(100, 8), direct=True))
    metas.append(TensorMeta("lm_head", (100, 8), "float32", alias_of="model.embed"))
    plan = TransferSchedule.build(metas, bucket_size=16 << 10)
    back = TransferSchedule.from_json(plan.to_json())
    assert back == plan and len(back.buckets) > 1
    bad = json.loads(plan.to_json())
    bad["buckets"][0]["tensors"][0]["offset"] = bad["buckets"][0]["nbytes"]
    with pytest.raises(ValueError):
        TransferSchedule.from_json(json.dumps(bad))
    bad = json.loads(plan.to_json())
    bad["direct"][0]["dtype"] = "object"
    with pytest.raises(ValueError):
        TransferSchedule.from_json(json.dumps(bad))
    with pytest.raises(ValueError):
        TransferSchedule.from_json(json.dumps({"version": 2}))


def test_sync_into_an_engine_that_stores_replicated_kv_heads():
    """Three query heads per K/V head: the engine stores every K/V head three times, the
    trainer sends (and /weights_info lists) the checkpoint's two."""
    from arcticinference_b200.models.loader import load_llama_state
    from arcticinference_b200.server.weight_sync.receiver import engine_weights_info
    over = {"hf_overrides": {"num_attention_heads": 6, "num_key_value_heads": 2, "hidden_size": 384,
                             "qkv_bias": True}}
    eng = engine("llama-tiny", **over)
    cfg = eng.config.model
    assert (cfg.num_key_value_heads, cfg.checkpoint_kv_heads) == (6, 2)
    D = cfg.head_dim
    state = {}
    for name, t in random_llama_state(cfg, 77, 0.05, "cpu", torch.bfloat16):
        if ".k_proj." in name or ".v_proj." in name:          # the trainer's two heads
            t = t.reshape(2, 3, D, *t.shape[1:])[:, 0].reshape(2 * D, *t.shape[1:]).contiguous()
        state[name] = t
    info = {d["name"]: tuple(d["shape"]) for d in engine_weights_info(eng)}
    assert all(info[n] == tuple(t.shape) for n, t in state.items())
    before = greedy(eng)
    p = port()
    sender = WeightSender(state, device="cpu", direct_names=["model.embed_tokens.weight", "lm_head.weight"])
    th = sender.start([{"master_addr": "127.0.0.1", "master_port": p, "replica_ids": [0]}],
                      bucket_size=1 << 20, timeout=60)
    res = engine_sync_weights(eng, {"master_addr": "127.0.0.1", "master_port": p, "timeout": 60})
    sender.join(th)
    assert res["incomplete_layers"] == []
    ref = engine("llama-tiny", **over)
    load_llama_state(ref.runner.model, state.items())
    after = greedy(eng)
    assert after == greedy(ref) and after != before


@pytest.mark.parametrize("reverse", [False, True])
def test_reference_named_channel_and_helpers(reverse, tmp_path):
    """The names a trainer written against the reference imports."""
    import threading
    from arcticinference_b200.server import (ModelConfig as SM, NCCLEngine, Pipeline, ReplicaPool,  # noqa: F401
                                             WeightInfo, build_weights_info, ensure_ray)
    from arcticinference_b200.server.weight_sync import (cleanup_shm, load_spec_checkpoint,
                                                         load_weights_from_shm, save_weights_to_shm,
                                                         spec_bucket_size)
    from arcticinference_b200.utils.safetensors_io import write_safetensors
    assert ensure_ray() is None
    g = torch.Generator().manual_seed(1)
    weights = {"a.weight": torch.randn(300, 70, generator=g).to(torch.bfloat16),
               "b.bias": torch.randn(70, generator=g), "c": torch.arange(10, dtype=torch.int64)}
    weights["tied"] = weights["a.weight"]
    p = port()
    got, stats = {}, {}

    def recv():
        eng = NCCLEngine("127.0.0.1", p, rank=1, world_size=2, device="cpu", reverse=reverse, timeout=60)
        for name, t in eng.receive_weights():
            got[name] = t if isinstance(t, str) else t.clone()
        eng.destroy()

    th = threading.Thread(target=recv)
    th.start()
    eng = NCCLEngine("127.0.0.1", p, rank=0, world_size=2, device="cpu", bucket_size=16 << 10,
                     reverse=reverse, timeout=60)
    stats = eng.send_weights(weights.items())
    eng.destroy()
    th.join(60)
    assert stats["num_tensors"] == 4 and stats["num_buckets"] >= 2
    for n in ("a.weight", "b.bias", "c"):
        assert torch.equal(got[n], weights[n])
    assert got["tied"] == "a.weight" or torch.equal(got["tied"], weights["a.weight"])

    # names, shapes and dtypes from safetensors headers; speculator checkpoints; shm hand-over
    write_safetensors(str(tmp_path / "model.safetensors"),
                      {"speculator.head.0.weight": weights["a.weight"], "speculator.ln": weights["b.bias"]})
    infos = {i.name: i for i in build_weights_info(str(tmp_path))}
    w = infos["speculator.head.0.weight"]
    assert tuple(w.shape) == (300, 70) and w.dtype == torch.bfloat16 and w.nbytes == 300 * 70 * 2
    assert WeightInfo.from_dict(w.to_dict()).shape == w.shape
    spec = load_spec_checkpoint(str(tmp_path))
    assert set(spec) == {"head.0.weight", "ln"} and 300 * 70 * 2 <= spec_bucket_size(spec) <= 256 << 20
    key = "t%d" % p
    save_weights_to_shm({"x": weights["b.bias"]}, key, shm_dir=str(tmp_path))
    assert torch.equal(load_weights_from_shm(key, shm_dir=str(tmp_path))["x"], weights["b.bias"])
    cleanup_shm(key, shm_dir=str(tmp_path))
    assert not [f for f in os.listdir(tmp_path) if key in f]


def test_sender_schedule_deals_targets_to_trainer_ranks():
    from arcticinference_b200.server.weight_sync import SenderSchedule, TransferGroup
    # 8 trainer ranks, 4 replicas of TP 2: one target each
    s = TransferSchedule.build("fsdp", 8, 4, 2)               # the reference's call
    assert isinstance(s, SenderSchedule) and s.num_groups == 8
    assert [g.targets for g in s.groups[:3]] == [[(0, 0)], [(0, 1)], [(1, 0)]]
    assert s.port_for_target(3, 1, 5000) == 5007 and s.ports_of(7, 5000) == [5007]
    # 4 trainer ranks for the same 8 targets: two each, round-robin
    s = SenderSchedule.build("dp", 4, 4, 2)
    assert [g.targets for g in s.groups] == [[(0, 0), (2, 0)], [(0, 1), (2, 1)],
                                             [(1, 0), (3, 0)], [(1, 1), (3, 1)]]
    assert s.groups[2].replica_ids == [1, 3] and s.groups[0].world_size == 2
    assert s.active_sender_ranks == [0, 1, 2, 3] and s.targets_of(9) == []
    covered = sorted(t for g in s.groups for t in g.targets)
    assert covered == [(r, t) for r in range(4) for t in range(2)]
    # more trainer ranks than targets: dp / fsdp leave the rest idle, zero3 keeps them in step
    assert SenderSchedule.build("dp", 8, 1, 2).num_groups == 2
    z = TransferSchedule.build(training_sharding="zero3", training_gpus=8, inference_replicas=1,
                               inference_tp=2)
    assert z.num_groups == 8 and [len(g.targets) for g in z.groups] == [1, 1, 0, 0, 0, 0, 0, 0]
    with pytest.raises(ValueError, match="zero3"):
        SenderSchedule.build("zero3", 4, 4, 2)
    with pytest.raises(ValueError, match="training_sharding"):
        SenderSchedule.build("pp", 4, 4, 2)
    assert isinstance(s.groups[0], TransferGroup)


def test_two_trainer_ranks_feed_two_replicas_by_plan():
    """Each trainer rank opens the channels the plan gives it; every replica is updated."""
    from arcticinference_b200.server.weight_sync import SenderSchedule
    plan = SenderSchedule.build("dp", 2, 2, 1)
    engines = [engine(), engine()]
    before = [greedy(e) for e in engines]
    state = new_state(seed=321)
    base = port()
    senders, threads = [], []
    for rank in plan.active_sender_ranks:
        s = WeightSender(state, device="cpu")
        senders.append(s)
        threads.append(s.start_ports("127.0.0.1", plan.ports_of(rank, base), bucket_size=1 << 20,
                                     timeout=60))
    results = [None, None]

    def recv(i):
        results[i] = engine_sync_weights(engines[i], {"master_addr": "127.0.0.1",
                                                      "master_port": plan.port_for_target(i, 0, base),
                                                      "timeout": 60})

    rts = [threading.Thread(target=recv, args=(i,)) for i in range(2)]
    [t.start() for t in rts]
    [t.join(60) for t in rts]
    for s, th in zip(senders, threads):
        s.join(th)
    assert all(r["incomplete_layers"] == [] for r in results)
    after = [greedy(e) for e in engines]
    assert after[0] == after[1] and after[0] != before[0]
