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

METRIC = "combined tok/s (prompt+generated), Llama-3.1-8B shift-parallel serving"

# Reference arm: which way of running the reference to try first for each GPU count (the rungs
# are described in baseline/run_reference.py); the others follow in order if it fails.
REFERENCE_RUNGS = ("plugin", "vllm-tp", "vllm-dp")
# seconds; together they stay inside the half hour a caller may give the whole arm
REFERENCE_RUNG_TIMEOUT_S = {"plugin": 420, "vllm-tp": 900, "vllm-dp": 400}


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
    ap.add_argument("--shift-parallel-threshold", type=int, default=None,
                    help="default: each arm's own default (this engine 128, the reference 512)")
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


def _run_bounded(cmd, env, log, limit_s) -> int:
    """Run a child in its own process group with stdout and stderr in ``log``; on expiry the
    whole group is ended (vLLM's engine and worker processes included). Returns its exit code,
    -1 after a timeout."""
    import signal
    with open(log, "w") as lf:
        p = subprocess.Popen(cmd, env=env, stdout=lf, stderr=subprocess.STDOUT,
                             start_new_session=True)
        try:
            return p.wait(timeout=limit_s)
        except subprocess.TimeoutExpired:
            for sig in (signal.SIGTERM, signal.SIGKILL):
                try:
                    os.killpg(p.pid, sig)
                except ProcessLookupError:
                    break
                try:
                    p.wait(timeout=20)
                    break
                except subprocess.TimeoutExpired:
                    continue
            return -1


def run_reference(args, rank, local_rank):
    """The unmodified reference (baseline/_ref) on the image's vLLM, in a child process whose
    environment carries nothing of the launcher's rendezvous; none of this package is imported
    on that path. Only rank 0 gets here: vLLM starts its own worker per GPU."""
    runner = os.path.join(REPO, "baseline", "run_reference.py")
    if not os.path.isdir(os.path.join(REPO, "baseline", "_ref", "arctic_inference")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref holds no copy of the reference"}))
        return 0
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK",
                        "GROUP_WORLD_SIZE", "ROLE_RANK", "ROLE_NAME", "ROLE_WORLD_SIZE",
                        "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS", "PYTHONPATH")
           and not k.startswith("TORCHELASTIC_")}
    rungs = list(REFERENCE_RUNGS)
    first = os.environ.get("AB200_REFERENCE_RUNG")
    if first is None:
        try:
            with open(os.path.join(REPO, "baseline", "reference_rungs.json")) as f:
                first = json.load(f).get(str(args.gpus))
        except (OSError, ValueError):
            first = None
    if first in rungs:
        rungs.remove(first)
        rungs.insert(0, first)
    if args.gpus == 1:
        rungs = [r for r in rungs if r != "vllm-dp"]
    failures = []
    for rung in rungs:
        cmd = [sys.executable, runner, "--rung", rung, "--gpus", str(args.gpus),
               "--steps", str(args.steps), "--warmup", str(args.warmup),
               "--requests-per-gpu", str(args.requests_per_gpu),
               "--input-len", str(args.input_len), "--output-len", str(args.output_len),
               "--shift-parallel-threshold", str(args.shift_parallel_threshold or 512),
               "--quantization", str(args.quantization)]
        if args.max_num_batched_tokens:
            cmd += ["--max-num-batched-tokens", str(args.max_num_batched_tokens)]
        clocks = ClockSampler(enabled=not args.no_clocks)
        clocks.start()
        log = os.path.join(REPO, "gpurun_out", "reference_%s_n%d.log" % (rung, args.gpus))
        result_file = log[:-4] + ".json"
        os.makedirs(os.path.dirname(log), exist_ok=True)
        if os.path.exists(result_file):
            os.remove(result_file)
        cmd += ["--result", result_file, "--stack-dump-after", "600"]
        rc = _run_bounded(cmd, env, log, REFERENCE_RUNG_TIMEOUT_S[rung])
        clock_info = clocks.stop(local_rank)
        res = None
        try:
            with open(result_file) as f:
                res = json.loads(f.read())
        except (OSError, ValueError):
            pass
        if rc != 0 or res is None:
            tail = ""
            try:
                with open(log) as lf:
                    tail = [l for l in lf.read().splitlines() if l.strip()][-1][-300:]
            except (OSError, IndexError):
                pass
            failures.append({"rung": rung, "rc": rc, "last_line": tail})
            continue
        n_req = args.requests_per_gpu * args.gpus
        line = {
            "impl": "reference", "metric": METRIC, "value": res["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8-weights/bf16-activations (vLLM dynamic fp8)",
            "data": "synthetic (uniform-random token ids, random-init weights)",
            "p50_ttft_ms": res["p50_ttft_ms"], "p50_tpot_ms": res["p50_tpot_ms"],
            "reference_class": {"plugin": "arctic_inference plug-in on vLLM %s" % res["vllm"],
                                "vllm-tp": "plain vLLM %s, tensor parallel" % res["vllm"],
                                "vllm-dp": "plain vLLM %s, one engine per GPU" % res["vllm"]}[rung],
            "config": {"model": "llama-3.1-8b", "global_batch": n_req, "seq_len": args.input_len,
                       "output_len": args.output_len, "parallelism": res["parallelism"],
                       "timing": "wall clock around LLM.generate (engine in vLLM's own processes)",
                       "rungs_failed": failures},
            "clocks": clock_info,
            "e2e": {"value": res["value"], "unit": "tokens/s",
                    "h2d_bytes_per_step": res["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": res["d2h_bytes_per_step"],
                    "ms_per_step": res["ms_per_step"]},
        }
        print(json.dumps(line))
        return 0
    print(json.dumps({"impl": "reference", "unavailable":
                      "vLLM could not serve the workload on this box: " + json.dumps(failures)}))
    return 0


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n_gpus = args.gpus

    if args.impl == "reference":
        return run_reference(args, rank, local_rank) if rank == 0 else 0

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
        kw.update(ulysses_sequence_parallel_size=n_gpus, enable_shift_parallel=True)
        if args.shift_parallel_threshold is not None:
            kw.update(shift_parallel_threshold=args.shift_parallel_threshold)
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
            "metric": METRIC,
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
