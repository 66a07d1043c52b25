"""Host-side cost of one decode step: scheduling, batch preparation and book-keeping for N
running requests, with the model's forward pass and LM head replaced by constants so that only
the engine's own Python and numpy work is timed. Runs on the CPU path (no GPU needed); the
scheduler, `ModelRunner.prepare` and `update_from_output` are the same code on a GPU.

    python benchmarks/host_step_cost.py --requests 1024 --prompt-len 2000 --steps 100

With run-ahead scheduling this work overlaps the previous step on the device, so it bounds the
step rate only where it exceeds the device time of a step. Prints one JSON line (milliseconds
per step).
"""

import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from arcticinference_b200 import LLM, SamplingParams  # noqa: E402


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-tiny", help="architecture (its size does not matter)")
    ap.add_argument("--requests", type=int, default=1024)
    ap.add_argument("--prompt-len", type=int, default=2000)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--block-size", type=int, default=16)
    a = ap.parse_args(argv)
    # requests admitted first keep decoding while the others are still being prefilled: give
    # every request enough tokens to outlast that and the timed steps
    out_len = a.steps + a.requests * a.prompt_len // 8192 + 64
    blocks = a.requests * ((a.prompt_len + out_len) // a.block_size + 2)
    llm = LLM(model=a.model, device="cpu", max_model_len=a.prompt_len + out_len + 1,
              max_num_seqs=a.requests, max_num_batched_tokens=8192, block_size=a.block_size,
              num_gpu_blocks_override=blocks, async_scheduling=True, enable_prefix_caching=False)
    eng = llm.engine
    model = eng.runner.model
    H, V = model.cfg.hidden_size, model.cfg.vocab_size
    model.forward = lambda batch, kv: torch.zeros(batch.logits_indices.numel(), H, dtype=torch.bfloat16)
    rows = {}

    def logits(hidden, fp32=False):
        n = hidden.shape[0]
        if n not in rows:
            t = torch.zeros(n, V, dtype=torch.bfloat16)
            t[:, 7] = 1.0
            rows[n] = t
        return rows[n]

    model.compute_logits = logits
    rng = np.random.default_rng(0)
    sp = SamplingParams(temperature=0, max_tokens=out_len, ignore_eos=True)
    for _ in range(a.requests):
        eng.add_request(None, rng.integers(0, V, size=a.prompt_len).tolist(), sp)
    while eng.scheduler.waiting or any(r.num_computed_tokens < r.num_prompt_tokens
                                       for r in eng.scheduler.running):
        eng.step()
    prepare, spent = eng.runner.prepare, [0.0]

    def timed(out):
        t = time.perf_counter()
        r = prepare(out)
        spent[0] += time.perf_counter() - t
        return r

    eng.runner.prepare = timed
    for k in ("t_schedule", "t_launch", "t_wait", "t_update"):
        eng.stats[k] = 0.0
    s0 = eng.stats["steps"]
    t0 = time.perf_counter()
    while eng.stats["steps"] - s0 < a.steps:
        eng.step()
    wall = time.perf_counter() - t0
    n = eng.stats["steps"] - s0
    ms = lambda x: round(x / n * 1e3, 3)
    res = {"case": "host_step_cost", "running_requests": len(eng.scheduler.running),
           "prompt_len": a.prompt_len, "steps": n, "ms_per_step": ms(wall),
           "schedule_ms": ms(eng.stats["t_schedule"]), "prepare_ms": ms(spent[0]),
           "launch_other_ms": ms(eng.stats["t_launch"] - spent[0]),
           "update_ms": ms(eng.stats["t_update"]), "wait_ms": ms(eng.stats["t_wait"])}
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
