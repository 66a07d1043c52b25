"""Pipeline parallelism on CPU ranks (gloo): whole-model stages must reproduce the one-rank
engine token for token, keep only their own layers and KV cache, and agree on the pool size."""

import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

from _mp_util import free_port as _free_port, result_or_child_failure as _result_or_child_failure

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROMPTS = [list(range(3, 70)), [9, 8, 7, 6, 5], list(range(100, 131))]
KW = dict(model="llama-tiny", device="cpu", num_gpu_blocks_override=64, block_size=16,
          max_model_len=512, hf_overrides={"num_hidden_layers": 5}, max_num_batched_tokens=48)


def _generate(llm):
    from arcticinference_b200 import SamplingParams
    sp = [SamplingParams(temperature=0, max_tokens=n, ignore_eos=True) for n in (9, 5, 12)]
    outs = llm.generate([{"prompt_token_ids": p} for p in PROMPTS], sp)
    return [o.outputs[0].token_ids for o in outs]


def _kw(model):
    return dict(KW, model=model)


def _worker(rank, world, port, q, model="llama-tiny"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    torch.set_num_threads(1)
    from arcticinference_b200 import LLM
    llm = LLM(pipeline_parallel_size=world, **_kw(model))
    toks = _generate(llm)
    m, r = llm.engine.runner.model, llm.engine.runner
    info = dict(rank=rank, toks=toks, layers=[i for i, lw in enumerate(m.layers) if lw is not None],
                kv=[i for i, k in enumerate(r.kv.k) if k is not None],
                blocks=llm.engine.num_blocks, stats=dict(r.pp.stats),
                run_ahead=llm.engine.stats["run_ahead_steps"])
    q.put(info)
    import torch.distributed as dist
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,model", [(2, "llama-tiny"), (3, "llama-tiny"), (2, "qwen3-tiny"),
                                         (2, "qwen2-tiny")])
def test_pipeline_stages_match_single_rank(world, model):
    from arcticinference_b200 import LLM
    want = _generate(LLM(**_kw(model)))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, model)) for r in range(world)]
    for p in procs:
        p.start()
    infos = [_result_or_child_failure(q, procs, 300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    infos.sort(key=lambda d: d["rank"])
    covered = []
    for d in infos:
        assert d["toks"] == want                    # every stage's scheduler saw the same tokens
        assert d["layers"] == d["kv"] and d["layers"]
        covered += d["layers"]
        assert d["blocks"] == infos[0]["blocks"]
    assert covered == list(range(5))               # each layer on exactly one stage, in order
    assert infos[0]["stats"]["send"] > 0 and infos[0]["stats"]["recv"] == 0
    assert infos[-1]["stats"]["recv"] > 0 and infos[-1]["stats"]["send"] == 0
    assert infos[0]["run_ahead"] > 0                # the next step is queued behind the ids' broadcast


def test_pipeline_refuses_what_it_cannot_serve():
    from arcticinference_b200.config import EngineArgs
    with pytest.raises(NotImplementedError):
        EngineArgs(model="llama-tiny", pipeline_parallel_size=2,
                   tensor_parallel_size=2).create_engine_config()
    with pytest.raises(NotImplementedError):
        EngineArgs(model="llama-tiny", pipeline_parallel_size=2,
                   speculative_config={"method": "suffix"}).create_engine_config()
    with pytest.raises(ValueError):
        EngineArgs(model="llama-tiny-swiftkv", pipeline_parallel_size=2).create_engine_config()
