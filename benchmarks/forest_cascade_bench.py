"""Decode steps of parallel samples that share one long prompt, with and without forest cascade
attention (the shared prefix's K/V read once per group instead of once per sample; reference:
arctic_inference/vllm/attention/flash_attn_forest_cascade.py:304-319 for the gates,
:1004-1026 for the two-pass call).

    python benchmarks/forest_cascade_bench.py --prompt-len 8192 --samples 64

One engine per arm, same weights and seed: the prompt is prefilled once, its `--samples`
continuations decode together, and `--steps` decode steps are timed on the device (CUDA
events around the loop, after `--warmup` steps). Prints one JSON line.
"""

import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from arcticinference_b200 import LLM, SamplingParams  # noqa: E402


def run(arm: str, a) -> dict:
    kw = dict(model=a.model, max_model_len=a.prompt_len + a.steps + a.warmup + 64,
              max_num_batched_tokens=8192, quantization=a.quantization, seed=0)
    if arm == "cascade":
        kw["forest_cascade_attn_configs"] = "{}"
    llm = LLM(**kw)
    eng = llm.engine
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 32000, size=a.prompt_len).tolist()
    sp = SamplingParams(n=a.samples, temperature=1.0, seed=1, ignore_eos=True,
                        max_tokens=a.steps + a.warmup + 8)
    eng.add_request(None, prompt, sp)
    # prefill, fan-out and the first decode steps
    guard = 0
    while eng.stats["generation_tokens"] < a.samples * a.warmup and guard < 10000:
        eng.step()
        guard += 1
    torch.cuda.synchronize()
    s0 = eng.stats["steps"]
    c0 = eng.runner.cascade_steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    while eng.stats["steps"] - s0 < a.steps:
        eng.step()
    e1.record()
    torch.cuda.synchronize()
    n = eng.stats["steps"] - s0
    res = {"ms_per_decode_step": e0.elapsed_time(e1) / n, "steps": n,
           "cascade_steps": eng.runner.cascade_steps - c0}
    for r in list(eng.scheduler.running):
        eng.abort_request(r.parent_id or r.request_id)
    del llm, eng
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--quantization", default="fp8")
    ap.add_argument("--prompt-len", type=int, default=8192)
    ap.add_argument("--samples", type=int, default=64)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=8)
    a = ap.parse_args()
    plain = run("plain", a)
    casc = run("cascade", a)
    print(json.dumps({"case": "forest_cascade_decode", "model": a.model, "prompt_len": a.prompt_len,
                      "samples": a.samples, "plain": plain, "cascade": casc,
                      "speedup": plain["ms_per_decode_step"] / casc["ms_per_decode_step"]}))


if __name__ == "__main__":
    main()
