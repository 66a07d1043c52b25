"""Run-ahead (asynchronous) scheduling must not change any output: the next decode step is
queued before the host has read the previous step's tokens, with the sampled tokens handed
over on the device."""

import asyncio

import pytest

from arcticinference_b200 import LLM, SamplingParams
from arcticinference_b200.config import EngineArgs
from arcticinference_b200.engine.async_llm import AsyncLLM

KW = dict(model="llama-tiny", device="cpu", block_size=16, max_model_len=256)
PROMPTS = [[5, 9, 200, 17, 3], [77] * 40, [1, 2, 3], list(range(10, 90)), [4, 4, 4, 4]]


def _run(async_on, sp, prompts=PROMPTS, blocks=256, **kw):
    llm = LLM(async_scheduling=async_on, num_gpu_blocks_override=blocks, **KW, **kw)
    outs = llm.generate(prompts, sp)
    return [[c.token_ids for c in o.outputs] for o in outs], [o.outputs[0].finish_reason for o in outs], llm


def test_greedy_outputs_identical_and_steps_overlap():
    sp = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True) for n in (12, 30, 1, 17, 25)]
    a, fa, _ = _run(False, sp)
    b, fb, llm = _run(True, sp)
    assert a == b and fa == fb
    assert llm.engine.stats["run_ahead_steps"] > 15          # most decode steps ran ahead
    assert llm.engine._pending is None and not llm.engine.has_unfinished_requests()


def test_token_dependent_stop_and_sampling():
    base, _, _ = _run(False, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    # a token that the first request produces in the middle of its output stops it there
    stop = base[0][0][7]
    sp = SamplingParams(temperature=0.0, max_tokens=40, stop_token_ids=[stop])
    a, fa, _ = _run(False, sp)
    b, fb, _ = _run(True, sp)
    assert a == b and fa == fb and "stop" in fa
    assert len(a[0][0]) <= 8
    # seeded sampling, several samples per prompt
    sp = SamplingParams(temperature=0.9, seed=11, n=2, max_tokens=15, ignore_eos=True)
    a, _, _ = _run(False, sp)
    b, _, llm = _run(True, sp)
    assert a == b and llm.engine.stats["run_ahead_steps"] > 5


def test_preemption_under_run_ahead():
    sp = SamplingParams(temperature=0.0, max_tokens=60, ignore_eos=True)
    prompts = [[i + 1] * 30 for i in range(6)]
    a, _, _ = _run(False, sp, prompts, blocks=24)             # too few blocks for all six
    b, _, llm = _run(True, sp, prompts, blocks=24)
    assert a == b and all(len(x[0]) == 60 for x in b)


def test_streaming_with_late_arrivals():
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    want, _, _ = _run(False, sp)

    async def main():
        llm = AsyncLLM.from_engine_args(EngineArgs(async_scheduling=True, num_gpu_blocks_override=256,
                                                   **{k: v for k, v in KW.items() if k != "device"}),
                                        device="cpu").start()
        try:
            async def one(p, delay):
                await asyncio.sleep(delay)
                last, n_parts = None, 0
                async for out in llm.generate(p, sp):
                    assert -1 not in out.outputs[0].token_ids     # no placeholder ever leaks
                    last, n_parts = out, n_parts + 1
                return last.outputs[0].token_ids, n_parts
            res = await asyncio.gather(*[one(p, 0.02 * i) for i, p in enumerate(PROMPTS)])
            assert [[r[0]] for r in res] == want
            assert all(r[1] >= 10 for r in res)
            assert llm.engine.stats["run_ahead_steps"] > 0
            # abort in the middle of a run-ahead stretch
            got = []
            async for out in llm.generate([9, 8, 7], SamplingParams(temperature=0.0, max_tokens=200,
                                                                   ignore_eos=True), "x"):
                got.append(out)
                if len(got) == 5:
                    await llm.abort("x")
            assert len(got[-1].outputs[0].token_ids) < 200
            assert (await llm.generate_final([1, 2, 3], sp)).outputs[0].token_ids == want[2][0]
        finally:
            llm.shutdown()
    asyncio.run(main())


def test_mixed_steps_run_ahead_with_chunked_prompts():
    """Prompt chunks, prompts that complete inside a step and admissions all run ahead: with
    a small token budget the long prompts are cut into chunks that share steps with the
    decodes of the short ones."""
    prompts = [list(range(10, 150)), [7, 8, 9], list(range(30, 120)), [5] * 70, [1, 2]]
    sp = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True) for n in (9, 40, 1, 22, 33)]
    kw = dict(max_num_batched_tokens=48, max_num_seqs=4)
    a, fa, ref = _run(False, sp, prompts, **kw)
    b, fb, llm = _run(True, sp, prompts, **kw)
    assert a == b and fa == fb
    st = llm.engine.stats
    assert st["steps"] == ref.engine.stats["steps"]
    # nearly every step after the first was queued while its predecessor was still running
    assert st["run_ahead_steps"] >= st["steps"] - 3, st
    assert llm.engine._pending is None and not llm.engine.has_unfinished_requests()
    assert all(r.chunk_ahead == 0 and not r.provisional for r in llm.engine.scheduler.finished)


def test_mixed_steps_with_prefix_cache_and_few_blocks():
    shared = list(range(200, 264))
    prompts = [shared + [i, i + 1, i + 2] * 5 for i in range(1, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)
    kw = dict(max_num_batched_tokens=64, enable_prefix_caching=True)
    a, fa, _ = _run(False, sp, prompts, blocks=20, **kw)
    b, fb, llm = _run(True, sp, prompts, blocks=20, **kw)
    assert a == b and fa == fb and all(len(x[0]) == 30 for x in b)
    assert llm.engine.stats["run_ahead_steps"] > 20


def test_full_distribution_requests_do_not_run_ahead():
    sp = [SamplingParams(temperature=0.8, top_p=0.9, seed=3, max_tokens=12, ignore_eos=True),
          SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)]
    a, _, _ = _run(False, sp, PROMPTS[:2])
    b, _, llm = _run(True, sp, PROMPTS[:2])
    assert a == b
    assert llm.engine.stats["run_ahead_steps"] == 0


@pytest.mark.parametrize("seed", range(16))
def test_random_workloads_are_unchanged_by_run_ahead(seed):
    """Random prompt lengths, output lengths, token budgets and cache sizes (small enough to
    force chunking and, for some seeds, preemption): same tokens, same finish reasons, same
    number of engine steps with and without run-ahead."""
    import random
    rng = random.Random(1234 + seed)
    n = rng.randint(3, 9)
    prompts = [[rng.randrange(3, 900) for _ in range(rng.randint(1, 120))] for _ in range(n)]
    sp = [SamplingParams(temperature=0.0 if rng.random() < 0.7 else 0.8, seed=rng.randrange(100),
                         max_tokens=rng.randint(1, 40), ignore_eos=rng.random() < 0.8)
          for _ in range(n)]
    kw = dict(max_num_batched_tokens=rng.choice([16, 48, 128, 512]),
              max_num_seqs=rng.choice([2, 4, 16]),
              enable_prefix_caching=rng.random() < 0.5)
    blocks = rng.choice([20, 32, 256])
    a, fa, ref = _run(False, sp, prompts, blocks=blocks, **kw)
    b, fb, llm = _run(True, sp, prompts, blocks=blocks, **kw)
    assert a == b and fa == fb, (kw, blocks)
    assert llm.engine.stats["run_ahead_steps"] > 0
    assert llm.engine.kv_manager.usage == ref.engine.kv_manager.usage


def test_streaming_with_chunked_prompts_and_arrivals_mid_prefill():
    prompts = [list(range(10, 130)), [3, 4, 5], list(range(200, 290)), [8] * 50]
    sp = SamplingParams(temperature=0.0, max_tokens=18, ignore_eos=True)
    want, _, _ = _run(False, sp, prompts, max_num_batched_tokens=32)

    async def main():
        llm = AsyncLLM.from_engine_args(
            EngineArgs(async_scheduling=True, num_gpu_blocks_override=256, max_num_batched_tokens=32,
                       **{k: v for k, v in KW.items() if k != "device"}), device="cpu").start()
        try:
            async def one(p, delay):
                await asyncio.sleep(delay)
                last = None
                async for out in llm.generate(p, sp):
                    assert -1 not in out.outputs[0].token_ids
                    last = out
                return last.outputs[0].token_ids
            res = await asyncio.gather(*[one(p, 0.01 * i) for i, p in enumerate(prompts)])
            assert [[r] for r in res] == want
            assert llm.engine.stats["run_ahead_steps"] > 10
        finally:
            llm.shutdown()
    asyncio.run(main())
