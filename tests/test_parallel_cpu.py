"""Multi-rank engine logic on CPU ranks (gloo): Ulysses SP, full TP, shift parallelism and
TP x SP grids must reproduce the single-rank engine's logits."""

import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from _mp_util import free_port as _free_port, result_or_child_failure as _result_or_child_failure

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


PROMPTS = [list(range(3, 70)), [9, 8, 7, 6, 5], list(range(100, 131))]


def _run_engine(llm, steps=3):
    """Return logits of the sampled rows for the first ``steps`` engine steps."""
    from arcticinference_b200 import SamplingParams
    eng = llm.engine
    for p in PROMPTS:
        eng.add_request(None, p, SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
    outs = []
    modes = []
    for _ in range(steps):
        out = eng.scheduler.schedule()
        batch, rows = eng.runner.prepare(out)
        with torch.inference_mode():
            h = eng.runner.model.forward(batch, eng.runner.kv)
            logits = eng.runner.model.compute_logits(h)
            if eng.comm is not None and eng.comm.ways > 1:
                logits = eng.comm.gather_vocab(logits, eng.config.model.vocab_size)
        outs.append(logits.float().clone())
        modes.append(batch.mode)
        # teacher forcing: feed fixed tokens, so that a near-tie in the arg-max of one run
        # cannot send the two engines down different continuations
        new = {}
        for i, (s, rr) in enumerate(zip(out.scheduled, rows)):
            if s.samples:
                new[s.request.request_id] = [(17 * len(outs) + 5 * i + 3) % 1000]
        eng.scheduler.update_from_output(out, new)
    return outs, modes


def _full_weights(model_name, seed=0):
    from arcticinference_b200 import LLM
    llm = LLM(model=model_name, device="cpu", num_gpu_blocks_override=64, block_size=16,
              max_model_len=512, seed=seed)
    return llm


def _worker(rank, world, port, tp, sp, shift, model_name, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    torch.set_num_threads(1)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from arcticinference_b200 import LLM
    from arcticinference_b200.parallel.comm import Communicator
    comm = Communicator(tp, sp, None)
    llm = LLM(model=model_name, device="cpu", comm=comm, num_gpu_blocks_override=64, block_size=16,
              max_model_len=512, tensor_parallel_size=tp, ulysses_sequence_parallel_size=sp,
              enable_shift_parallel=shift, shift_parallel_threshold=8)
    outs, modes = _run_engine(llm)
    if rank == 0:
        q.put(([o.numpy() for o in outs], modes))
    dist.barrier()
    dist.destroy_process_group()


def _launch(tp, sp, shift, model_name):
    world = tp * sp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tp, sp, shift, model_name, q))
             for r in range(world)]
    for p in procs:
        p.start()
    res = _result_or_child_failure(q, procs, 300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return res


@pytest.mark.parametrize("tp,sp,shift,model", [
    (1, 2, False, "llama-tiny"),
    (2, 1, False, "llama-tiny"),
    (1, 2, True, "llama-tiny"),
    (2, 2, True, "llama-tiny"),
    (1, 2, True, "llama-tiny-swiftkv"),
    (1, 2, True, "qwen3-tiny"),
    (2, 1, False, "qwen3-tiny"),
    (1, 2, True, "qwen2-tiny"),
    (2, 1, False, "qwen2-tiny"),
])
def test_parallel_modes_match_single_rank(tp, sp, shift, model):
    ref_llm = _full_weights(model)
    ref_outs, _ = _run_engine(ref_llm)
    outs, modes = _launch(tp, sp, shift, model)
    if shift:
        assert "sp" in modes and "tp" in modes   # prefill in SP mode, decode in TP mode
    for a, b in zip(outs, ref_outs):
        a = torch.from_numpy(a)
        assert a.shape == b.shape
        err = (a - b).abs().max().item()
        assert err < 0.05 * max(1.0, b.abs().max().item()), (err, modes)


def _generate_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    torch.set_num_threads(1)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from arcticinference_b200 import LLM, SamplingParams
    from arcticinference_b200.parallel.comm import Communicator
    comm = Communicator(1, world, None)
    prompts = [list(range(3, 100)), [9, 8, 7, 6, 5], list(range(100, 160)), [4] * 33]
    sp = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True) for n in (10, 25, 1, 14)]
    res = []
    for async_on in (False, True):
        llm = LLM(model="llama-tiny", device="cpu", comm=comm, num_gpu_blocks_override=64,
                  block_size=16, max_model_len=512, ulysses_sequence_parallel_size=world,
                  enable_shift_parallel=True, shift_parallel_threshold=8,
                  max_num_batched_tokens=40, async_scheduling=async_on)
        outs = llm.generate(prompts, sp)
        res.append(([o.outputs[0].token_ids for o in outs], llm.engine.stats["run_ahead_steps"],
                    dict(llm.engine.runner.mode_counts)))
    every = [None] * world
    dist.all_gather_object(every, res[1][0])
    # log-probabilities over a vocabulary that is split between the ranks
    sp2 = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True, logprobs=2, prompt_logprobs=0)
    par = llm.generate(prompts[:1], sp2)[0]
    lp = (par.outputs[0].token_ids, par.outputs[0].logprobs, par.prompt_logprobs)
    if rank == 0:
        one = LLM(model="llama-tiny", device="cpu", num_gpu_blocks_override=64, block_size=16,
                  max_model_len=512).generate(prompts[:1], sp2)[0]
        q.put((res, every, lp, (one.outputs[0].token_ids, one.outputs[0].logprobs,
                                one.prompt_logprobs)))
    dist.barrier()
    dist.destroy_process_group()


def test_run_ahead_on_two_ranks_with_chunked_prompts_and_mode_shifts():
    """Both ranks schedule on their own (SPMD): with run-ahead stepping, chunked prompts and
    shifts between the two modes they must still agree with each other and with synchronous
    stepping."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_generate_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res, every, lp_two_ranks, lp_one_rank = _result_or_child_failure(q, procs, 300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    (sync_tokens, sync_ahead, _), (async_tokens, async_ahead, modes) = res
    assert sync_tokens == async_tokens
    assert sync_ahead == 0 and async_ahead > 10
    assert modes["sp"] > 0 and modes["tp"] > 0
    assert all(e == async_tokens for e in every)
    # prompt positions are teacher-forced, so they compare across layouts; generated tokens
    # can part ways at a near-tie of this random model, so only the first one is compared
    a, b = lp_two_ranks[2][1:], lp_one_rank[2][1:]
    assert len(a) == len(b) and all(abs(x - y) < 5e-2 for x, y in zip(a, b))
    assert lp_two_ranks[0][0] == lp_one_rank[0][0]
    assert abs(lp_two_ranks[1][0] - lp_one_rank[1][0]) < 5e-2 and len(lp_two_ranks[1]) == 4


def _spec_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    torch.set_num_threads(1)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from arcticinference_b200 import LLM
    from arcticinference_b200.parallel.comm import Communicator
    comm = Communicator(world, 1, None)
    llm = LLM(model="llama-tiny", device="cpu", comm=comm, num_gpu_blocks_override=64, block_size=16,
              max_model_len=512, tensor_parallel_size=world, speculative_config=_SPEC)
    prop = llm.engine.runner.proposer
    h, tok = _spec_inputs(prop.cfg.input_hidden_dim)
    drafts = prop.propose(h, tok, 3)
    rows = prop.w["head.0.weight"].shape[0]
    from arcticinference_b200 import SamplingParams
    outs = llm.generate([{"prompt_token_ids": p} for p in PROMPTS[:2]],
                        SamplingParams(temperature=0, max_tokens=6, ignore_eos=True))
    toks = [o.outputs[0].token_ids for o in outs]
    if rank == 0:
        q.put((drafts.numpy(), rows, toks, llm.engine.stats["draft_tokens"]))
    dist.barrier()
    dist.destroy_process_group()


_SPEC = {"method": "arctic", "model": "random", "num_speculative_tokens": 3}


def _spec_inputs(dim):
    g = torch.Generator().manual_seed(5)
    return torch.randn(6, dim, generator=g).to(torch.bfloat16), torch.arange(6, dtype=torch.int64) * 7


def test_speculator_heads_sharded_by_vocabulary_draft_the_same_tokens():
    """Tensor-parallel ranks keep 1/W of each speculator LM head and exchange one
    (value, token) candidate per row; the drafts equal the single-rank speculator's."""
    from arcticinference_b200 import LLM
    ref = LLM(model="llama-tiny", device="cpu", num_gpu_blocks_override=64, block_size=16,
              max_model_len=512, speculative_config=_SPEC)
    prop = ref.engine.runner.proposer
    h, tok = _spec_inputs(prop.cfg.input_hidden_dim)
    want = prop.propose(h, tok, 3)
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_spec_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got, rows, toks, drafted = _result_or_child_failure(q, procs, 300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert rows == prop.cfg.vocab_size // world
    assert (got == want.numpy()).all(), (got, want)
    # and the two-rank engine generates with them (drafts verified and re-drafted in the step)
    from arcticinference_b200 import SamplingParams
    assert drafted > 0 and [len(t) for t in toks] == [6, 6]
    base = LLM(model="llama-tiny", device="cpu", num_gpu_blocks_override=64, block_size=16,
               max_model_len=512)
    want_toks = [o.outputs[0].token_ids for o in base.generate(
        [{"prompt_token_ids": p} for p in PROMPTS[:2]],
        SamplingParams(temperature=0, max_tokens=6, ignore_eos=True))]
    assert [t[0] for t in toks] == [t[0] for t in want_toks]
