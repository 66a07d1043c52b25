"""Prefill-only comparison of Ulysses sequence parallelism with tensor parallelism over the
same GPUs: a batch of long prompts, one generated token each, one mode per invocation.

The workload is the reference's Ulysses claim (projects/ulysses/README.md:5: time to first
token of long prompts, SP against TP over the same 8 GPUs): 8 prompts of 8192 uniform-random
tokens, Llama-3.1-8B, bf16. One process per GPU; the timed region is bracketed by a barrier
and a device synchronisation, timed with CUDA events, maximum over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29561 benchmarks/prefill_sp_vs_tp.py --mode sp
    python -m torch.distributed.run ... benchmarks/prefill_sp_vs_tp.py --mode tp
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mode", choices=["sp", "tp"], required=True)
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--quantization", default="none")
    ap.add_argument("--num-prompts", type=int, default=8)
    ap.add_argument("--input-len", type=int, default=8192)
    ap.add_argument("--max-num-batched-tokens", type=int, default=None,
                    help="default: the whole batch in one step")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--comm-backend", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)

    import numpy as np
    import torch
    import torch.distributed as dist
    from arcticinference_b200 import LLM, SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available() and a.device != "cpu"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    budget = a.max_num_batched_tokens or a.num_prompts * a.input_len
    quant = None if str(a.quantization).lower() in ("none", "bf16", "") else a.quantization
    kw = dict(model=a.model, max_model_len=a.input_len + 64, max_num_batched_tokens=budget,
              max_num_seqs=max(256, a.num_prompts), enable_prefix_caching=False,
              quantization=quant, comm_backend=a.comm_backend)
    if a.device:
        kw["device"] = a.device
    if world > 1:
        kw.update({"sp": dict(ulysses_sequence_parallel_size=world),
                   "tp": dict(tensor_parallel_size=world)}[a.mode])
    llm = LLM(**kw)
    vocab = llm.engine.config.model.vocab_size
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)

    def batch(seed):
        rng = np.random.default_rng(seed)            # the same prompts on every rank
        return [{"prompt_token_ids": rng.integers(0, vocab, size=a.input_len).tolist()}
                for _ in range(a.num_prompts)]

    def sync():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    for i in range(a.warmup):
        llm.generate(batch(100 + i), sp)
    times = []
    for i in range(a.iters):
        prompts = batch(200 + i)
        sync()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        llm.generate(prompts, sp)
        if cuda:
            e1.record()
        sync()
        ms = e0.elapsed_time(e1) if cuda else 1e3 * (time.perf_counter() - t0)
        t = torch.tensor([ms], dtype=torch.float64, device="cuda" if cuda else "cpu")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t[0]))
    if cuda:
        from arcticinference_b200 import ops
        ops.check_status()
    times.sort()
    med = times[len(times) // 2]
    tokens = a.num_prompts * a.input_len
    res = {"mode": a.mode if world > 1 else "single", "n_gpus": world, "model": a.model,
           "num_prompts": a.num_prompts, "input_len": a.input_len, "tokens_per_step": budget,
           "median_ms": med, "best_ms": times[0], "prefill_tokens_per_s": tokens / (med / 1e3),
           "comm_backend": a.comm_backend}
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
    return res


if __name__ == "__main__":
    main()
