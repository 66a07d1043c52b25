"""Reference arm of ``bench.py``: the headline serving benchmark run by the UNMODIFIED reference
(``arctic_inference`` as found under ``baseline/_ref``) as a plug-in of the vLLM that is installed
in the image, through vLLM's own public ``LLM(...).generate`` API.

Nothing of ``arcticinference_b200`` is imported here. The workload is the one ``bench.py`` gives
its own arm: waves of ``requests_per_gpu * N`` requests of ``input_len`` uniform-random prompt
tokens and ``output_len`` generated tokens (the reference's ``batch`` task,
tests/benchmarks/benchmark_utils.py:91-116), a Llama-3.1-8B architecture with random ("dummy")
weights quantised to fp8 by vLLM, one engine over N GPUs.

Rungs (``--rung``), tried by ``bench.py`` in this order until one completes:

``plugin``     vLLM + the Arctic Inference plug-in (``ARCTIC_INFERENCE_ENABLED=1``; for N > 1
               ``ulysses_sequence_parallel_size=N, enable_shift_parallel=True``: the reference's
               shift-parallel deployment, README.md:107-120 of the reference).
``vllm-tp``    plain vLLM of the image, ``tensor_parallel_size=N`` (the plug-in left off).
``vllm-dp``    N independent plain-vLLM engines, one per GPU, each serving its share of the wave.

The timed region is wall clock around ``LLM.generate`` (the engine runs in vLLM's own worker
processes, so there is no device event to bracket it with); the prompts are host lists and the
generated ids come back to the host, i.e. it is an end-to-end number.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

LLAMA_31_8B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "hidden_size": 4096,
    "intermediate_size": 14336,
    "num_hidden_layers": 32,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "vocab_size": 128256,
    "max_position_embeddings": 131072,
    "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
    "tie_word_embeddings": False,
    "torch_dtype": "bfloat16",
    "bos_token_id": 128000,
    "eos_token_id": 128001,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rung", default="plugin", choices=["plugin", "vllm-tp", "vllm-dp"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--requests-per-gpu", type=int, default=128)
    ap.add_argument("--input-len", type=int, default=2000)
    ap.add_argument("--output-len", type=int, default=250)
    ap.add_argument("--max-num-batched-tokens", type=int, default=None)
    ap.add_argument("--shift-parallel-threshold", type=int, default=512)
    ap.add_argument("--quantization", default="fp8")
    ap.add_argument("--seed-offset", type=int, default=0,
                    help="vllm-dp children: which share of the wave this engine serves")
    ap.add_argument("--share", type=int, default=1, help="vllm-dp children: number of shares")
    ap.add_argument("--result", default=None,
                    help="write the result line to this file (vLLM logs to stdout as well)")
    ap.add_argument("--stack-dump-after", type=int, default=0,
                    help="seconds after which the stacks of this process are dumped to stderr "
                         "(to see where a run that does not finish is waiting)")
    return ap.parse_args()


def emit(args, line: dict) -> None:
    text = json.dumps(line)
    if args.result:
        with open(args.result, "w") as f:
            f.write(text + "\n")
    print(text, flush=True)


def model_dir():
    d = os.path.join(tempfile.gettempdir(), "ab200_ref_llama31_8b")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(LLAMA_31_8B, f)
    return d


def run_dp(args):
    """N plain engines, one per GPU, run side by side; the wave is split evenly."""
    procs = []
    for i in range(args.gpus):
        env = dict(os.environ)
        env["CUDA_VISIBLE_DEVICES"] = str(i)
        cmd = [sys.executable, os.path.abspath(__file__), "--rung", "vllm-tp", "--gpus", "1",
               "--steps", str(args.steps), "--warmup", str(args.warmup),
               "--requests-per-gpu", str(args.requests_per_gpu),
               "--input-len", str(args.input_len), "--output-len", str(args.output_len),
               "--quantization", args.quantization, "--seed-offset", str(i),
               "--share", str(args.gpus),
               "--result", os.path.join(tempfile.gettempdir(), "ab200_ref_dp_%d.json" % i)]
        procs.append((subprocess.Popen(cmd, env=env), cmd[-1]))
    lines = []
    for p, result in procs:
        if p.wait() != 0:
            raise SystemExit("a data-parallel engine failed (exit %d)" % p.returncode)
        with open(result) as f:
            lines.append(json.loads(f.read()))
    ms = max(l["ms_per_step"] for l in lines)
    tokens = args.gpus * args.requests_per_gpu * (args.input_len + args.output_len)
    ttft = statistics.median(l["p50_ttft_ms"] for l in lines if l["p50_ttft_ms"] is not None)
    tpot = statistics.median(l["p50_tpot_ms"] for l in lines if l["p50_tpot_ms"] is not None)
    emit(args, {"rung": "vllm-dp", "value": tokens / (ms / 1000.0), "ms_per_step": ms,
                "p50_ttft_ms": ttft, "p50_tpot_ms": tpot,
                "h2d_bytes_per_step": sum(l["h2d_bytes_per_step"] for l in lines),
                "d2h_bytes_per_step": sum(l["d2h_bytes_per_step"] for l in lines),
                "vllm": lines[0]["vllm"], "parallelism": "dp%d" % args.gpus})


def main():
    args = parse_args()
    if args.rung == "vllm-dp":
        return run_dp(args)

    n = args.gpus
    if args.stack_dump_after > 0:
        import faulthandler
        faulthandler.dump_traceback_later(args.stack_dump_after, repeat=True, file=sys.stderr)
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    if args.rung == "plugin":
        os.environ["ARCTIC_INFERENCE_ENABLED"] = "1"
        os.environ["ARCTIC_INFERENCE_SKIP_VERSION_CHECK"] = "1"
        if REF not in sys.path:
            sys.path.insert(0, REF)
        os.environ["PYTHONPATH"] = REF + os.pathsep + os.environ.get("PYTHONPATH", "")
    else:
        os.environ["ARCTIC_INFERENCE_ENABLED"] = "0"

    import numpy as np
    import vllm
    from vllm import LLM, SamplingParams

    budget = args.max_num_batched_tokens or 8192 * n
    kw = dict(model=model_dir(), skip_tokenizer_init=True, load_format="dummy",
              dtype="bfloat16", max_model_len=args.input_len + args.output_len + 64,
              max_num_batched_tokens=budget, max_num_seqs=max(256, args.requests_per_gpu * n),
              enable_prefix_caching=False, disable_log_stats=False, seed=0,
              generation_config="vllm")
    if args.quantization not in ("none", "bf16", ""):
        kw["quantization"] = args.quantization
    parallelism = "single"
    if args.rung == "plugin" and n > 1:
        kw.update(ulysses_sequence_parallel_size=n, enable_shift_parallel=True,
                  shift_parallel_threshold=args.shift_parallel_threshold)
        parallelism = "sp%d<->tp%d shift" % (n, n)
    elif n > 1:
        kw.update(tensor_parallel_size=n)
        parallelism = "tp%d" % n
    llm = LLM(**kw)

    n_req = args.requests_per_gpu * n
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True,
                        detokenize=False)
    vocab = LLAMA_31_8B["vocab_size"]

    def make_wave(seed):
        rng = np.random.default_rng(seed * 1000 + args.seed_offset)
        return [{"prompt_token_ids": rng.integers(0, vocab, size=args.input_len).tolist()}
                for _ in range(n_req)]

    print("[run_reference] engine up, %d warm-up waves of %d requests" % (args.warmup, n_req),
          file=sys.stderr, flush=True)
    for w in range(args.warmup):
        t_w = time.perf_counter()
        llm.generate(make_wave(1000 + w), sp, use_tqdm=False)
        print("[run_reference] warm-up wave %d: %.1f s" % (w, time.perf_counter() - t_w),
              file=sys.stderr, flush=True)

    ttfts, tpots = [], []
    h2d = d2h = 0
    t0 = time.perf_counter()
    for k in range(args.steps):
        outs = llm.generate(make_wave(2000 + k), sp, use_tqdm=False)
        for o in outs:
            ids = o.outputs[0].token_ids
            h2d += 8 * len(o.prompt_token_ids)
            d2h += 8 * len(ids)
            m = getattr(o, "metrics", None)
            if m is not None and getattr(m, "first_token_latency", 0.0):
                ttfts.append(m.first_token_latency)
                if len(ids) > 1 and m.last_token_ts > m.first_token_ts:
                    tpots.append((m.last_token_ts - m.first_token_ts) / (len(ids) - 1))
    wall = time.perf_counter() - t0

    tokens = n_req * (args.input_len + args.output_len) * args.steps
    emit(args, {
        "rung": args.rung, "value": tokens / wall, "ms_per_step": 1000.0 * wall / args.steps,
        "p50_ttft_ms": 1000 * statistics.median(ttfts) if ttfts else None,
        "p50_tpot_ms": 1000 * statistics.median(tpots) if tpots else None,
        "h2d_bytes_per_step": h2d / args.steps, "d2h_bytes_per_step": d2h / args.steps,
        "vllm": vllm.__version__, "parallelism": parallelism})
    # vLLM's worker processes are torn down with the interpreter; leave without waiting for
    # destructors that have hung on some versions
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
