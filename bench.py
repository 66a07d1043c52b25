"""Headline benchmark: serving throughput of Llama-3.1-8B (random weights, synthetic
requests) through the public ``LLM.generate`` API, one engine spanning N GPUs with
shift parallelism (Ulysses SP=N for large steps, TP=N for small ones).

A "step" is one wave of ``requests_per_gpu * N`` requests, each a prompt of
``--input-len`` uniform-random tokens and ``--output-len`` generated tokens
(the reference's batch task is 2000 in / 250 out:
tests/benchmarks/benchmark_utils.py:91-116). The reported value is combined
(prompt + generated) tokens per second over the whole job; p50 TTFT / TPOT are
reported beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

REFERENCE_UNAVAILABLE = (
    "reference cannot be installed offline: its build needs nanobind==2.9.2 and grpcio-tools, "
    "neither is in the wheelhouse (pip install --no-index of the reference fails in cmake)")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", type=str, default="llama-3.1-8b")
    ap.add_argument("--quantization", type=str, default="fp8",
                    help='"fp8" (block-scaled fp8 weights, bf16 activations; the named config) or "none" (bf16)')
    ap.add_argument("--requests-per-gpu", type=int, default=128)
    ap.add_argument("--input-len", type=int, default=2000)
    ap.add_argument("--output-len", type=int, default=250)
    ap.add_argument("--max-num-batched-tokens", type=int, default=None,
                    help="token budget of one engine step; default 8192 per GPU, so that a step "
                         "gives every GPU the same work whatever N is")
    ap.add_argument("--shift-parallel-threshold", type=int, default=512)
    ap.add_argument("--speculative-config", type=str, default=None)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--no-clocks", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, enabled=True):
        self.proc = None
        self.enabled = enabled

    def start(self):
        if not self.enabled:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self, local_rank=0):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                if int(f[0]) != local_rank:
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return None
        busy = [c for c in sm if c > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n_gpus = args.gpus

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import numpy as np
    import torch

    if world != n_gpus:
        if world == 1 and n_gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node %d" % n_gpus)
    torch.cuda.set_device(local_rank)

    from arcticinference_b200 import LLM, SamplingParams, ops

    if args.max_num_batched_tokens is None:
        args.max_num_batched_tokens = 8192 * n_gpus
    quant = None if str(args.quantization).lower() in ("none", "bf16", "") else args.quantization
    kw = dict(model=args.model, max_model_len=args.input_len + args.output_len + 64,
              max_num_batched_tokens=args.max_num_batched_tokens,
              max_num_seqs=max(256, args.requests_per_gpu * n_gpus),
              enable_prefix_caching=False, enforce_eager=args.enforce_eager,
              quantization=quant, speculative_config=args.speculative_config)
    if n_gpus > 1:
        kw.update(ulysses_sequence_parallel_size=n_gpus, enable_shift_parallel=True,
                  shift_parallel_threshold=args.shift_parallel_threshold)
    llm = LLM(**kw)
    engine = llm.engine
    vocab = engine.config.model.vocab_size
    n_req = args.requests_per_gpu * n_gpus
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)

    def make_wave(seed):
        rng = np.random.default_rng(seed)  # same prompts on every rank
        return [{"prompt_token_ids": rng.integers(0, vocab, size=args.input_len).tolist()}
                for _ in range(n_req)]

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def run_wave(seed):
        outs = llm.generate(make_wave(seed), sp)
        return outs

    for w in range(args.warmup):
        run_wave(1000 + w)

    tokens_per_step = n_req * (args.input_len + args.output_len)

    # ---- device-timed region: K waves bracketed by CUDA events
    clocks = ClockSampler(enabled=(rank == 0 and not args.no_clocks))
    barrier()
    clocks.start()
    launches0 = ops.count_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ttfts, tpots = [], []
    ev0.record()
    for k in range(args.steps):
        for o in run_wave(2000 + k):
            if o.metrics.ttft is not None:
                ttfts.append(o.metrics.ttft)
            tp = o.metrics.tpot(len(o.outputs[0].token_ids))
            if tp is not None:
                tpots.append(tp)
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    launches = ops.count_launches() - launches0
    clock_info = clocks.stop(local_rank)

    # ---- end-to-end region: wall clock around the public API, including per-step
    # host->device staging of inputs (pinned) and device->host reads of sampled tokens
    engine.runner.h2d_total = 0
    engine.runner.d2h_total = 0
    steps0 = engine.stats["steps"]
    host0 = {k: engine.stats[k] for k in ("t_schedule", "t_launch", "t_wait", "t_update")}
    sync0 = engine.runner.sync_seconds
    barrier()
    t0 = time.perf_counter()
    for k in range(args.steps):
        run_wave(3000 + k)
    barrier()
    e2e_s = time.perf_counter() - t0
    e2e_steps = max(1, engine.stats["steps"] - steps0)
    # where the host spent the end-to-end region (rank 0), milliseconds per engine step
    host_ms = {k[2:]: 1000.0 * (engine.stats[k] - v) / e2e_steps for k, v in host0.items()}
    host_ms["device_wait"] = 1000.0 * (engine.runner.sync_seconds - sync0) / e2e_steps

    t = torch.tensor([dev_ms, e2e_s * 1000.0], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    ops.check_status()

    if rank == 0:
        value = tokens_per_step * args.steps / (dev_ms / 1000.0)
        e2e_value = tokens_per_step * args.steps / (e2e_ms / 1000.0)
        line = {
            "impl": "ours",
            "metric": "combined tok/s (prompt+generated), Llama-3.1-8B shift-parallel serving",
            "value": value, "unit": "tokens/s", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if not quant else "fp8-weights/bf16-activations",
            "data": "synthetic (uniform-random token ids, random-init weights)",
            "p50_ttft_ms": 1000 * statistics.median(ttfts) if ttfts else None,
            "p50_tpot_ms": 1000 * statistics.median(tpots) if tpots else None,
            "config": {
                "model": args.model, "global_batch": n_req, "seq_len": args.input_len,
                "output_len": args.output_len,
                "parallelism": ("sp%d<->tp%d shift" % (n_gpus, n_gpus)) if n_gpus > 1 else "single",
                "l2": "inputs larger than L2 (weights streamed every engine step)",
                "max_num_batched_tokens": args.max_num_batched_tokens,
                "engine_steps_per_wave": e2e_steps / args.steps,
                "host_ms_per_engine_step": {k: round(v, 3) for k, v in host_ms.items()},
                "mode_counts": dict(engine.runner.mode_counts),
            },
            "clocks": clock_info,
            "e2e": {"value": e2e_value, "unit": "tokens/s",
                    "h2d_bytes_per_step": getattr(engine.runner, "h2d_total", 0) / args.steps,
                    "d2h_bytes_per_step": getattr(engine.runner, "d2h_total", 0) / args.steps,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches,
        }
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
