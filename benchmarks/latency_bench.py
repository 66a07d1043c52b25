"""Single-stream latency: requests one at a time (concurrency 1), mean TTFT and TPOT.

The reference's ``single`` performance task (tests/benchmarks/benchmark_utils.py:104-116):
20 random prompts of 2000 tokens, 250 generated tokens each, one request in flight; it
reports the mean time to first token and the mean time per output token. ``bench.py`` at the
repository root is the ``batch`` task (throughput); this script is its latency counterpart.
One process per GPU; with N > 1 launch it under ``torch.distributed.run`` like ``bench.py``.

    python benchmarks/latency_bench.py [--model llama-3.1-8b] [--quantization fp8] \
        [--num-prompts 20] [--input-len 2000] [--output-len 250] [--gpus N] \
        [--speculative-config JSON]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--quantization", default="fp8")
    ap.add_argument("--num-prompts", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--input-len", type=int, default=2000)
    ap.add_argument("--output-len", type=int, default=250)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--shift-parallel-threshold", type=int, default=512)
    ap.add_argument("--speculative-config", default=None)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)

    import numpy as np
    import torch
    from arcticinference_b200 import LLM, SamplingParams

    rank = int(os.environ.get("RANK", "0"))
    if torch.cuda.is_available() and a.device is None:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    quant = None if str(a.quantization).lower() in ("none", "bf16", "") else a.quantization
    kw = dict(model=a.model, max_model_len=a.input_len + a.output_len + 64, quantization=quant,
              enable_prefix_caching=False, speculative_config=a.speculative_config)
    if a.device:
        kw["device"] = a.device
    if a.gpus > 1:
        kw.update(ulysses_sequence_parallel_size=a.gpus, enable_shift_parallel=True,
                  shift_parallel_threshold=a.shift_parallel_threshold)
    llm = LLM(**kw)
    vocab = llm.engine.config.model.vocab_size
    rng = np.random.default_rng(0)           # the same prompts on every rank
    sp = SamplingParams(temperature=0.0, max_tokens=a.output_len, ignore_eos=True)
    ttft, tpot, e2e = [], [], []
    for i in range(a.warmup + a.num_prompts):
        prompt = {"prompt_token_ids": rng.integers(0, vocab, size=a.input_len).tolist()}
        t0 = time.perf_counter()
        out = llm.generate([prompt], sp)[0]
        dt = time.perf_counter() - t0
        if i < a.warmup:
            continue
        m = out.metrics
        n = len(out.outputs[0].token_ids)
        if m.ttft is not None:
            ttft.append(m.ttft)
        tp = m.tpot(n)
        if tp is not None:
            tpot.append(tp)
        e2e.append(dt)
    res = {"task": "single", "model": a.model, "n_gpus": a.gpus, "num_prompts": a.num_prompts,
           "input_len": a.input_len, "output_len": a.output_len,
           "mean_ttft_ms": 1e3 * statistics.mean(ttft) if ttft else None,
           "mean_tpot_ms": 1e3 * statistics.mean(tpot) if tpot else None,
           "mean_e2el_ms": 1e3 * statistics.mean(e2e),
           "output_tokens_per_s": a.output_len / statistics.mean(e2e)}
    if rank == 0:
        print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
