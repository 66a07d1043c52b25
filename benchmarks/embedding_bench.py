"""Embedding throughput of one GPU: tokens/s through ``EmbeddingEngine.encode`` (token lists
on the host in, fp32 vectors on the host out), for short (50-token) and long (512-token)
sequences of uniform-random ids on a random-weight BERT-base. This is the workload of the
reference's embedding benchmark (benchmark/embedding/benchmark.py), which reports
tokens/s/GPU with one replica per GPU.

    python benchmarks/embedding_bench.py [--model bert-base] [--short 16384] [--long 2048]

The timed region covers host batching, the host->device copies of the token ids from pinned
memory, the encoder, pooling, and the device->host copies of the embeddings.
"""

import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from arcticinference_b200 import ops  # noqa: E402
from arcticinference_b200.embedding.engine import EmbeddingEngine  # noqa: E402


def run(engine, n_seqs, length, iters, warmup):
    rng = np.random.default_rng(0)
    # pre-tokenised inputs as they arrive from the wire: one int array per sequence
    seqs = list(rng.integers(0, engine.cfg.vocab_size, size=(n_seqs, length), dtype=np.int64))
    for _ in range(warmup):
        engine.encode(seqs[: max(64, n_seqs // 8)])
    torch.cuda.synchronize()
    l0 = ops.count_launches()
    t0 = time.perf_counter()
    for _ in range(iters):
        out = engine.encode(seqs)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / iters
    assert np.isfinite(out).all()
    cfg = engine.cfg
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    flops = n_seqs * length * L * (2.0 * H * (4 * H + 2 * I) + 4.0 * length * H)
    return {"length": length, "sequences": n_seqs, "seconds": dt,
            "tokens_per_s": n_seqs * length / dt, "sequences_per_s": n_seqs / dt,
            "model_tflops": flops / dt / 1e12, "launches": (ops.count_launches() - l0) // iters}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="bert-base")
    ap.add_argument("--short", type=int, default=16384, help="number of 50-token sequences")
    ap.add_argument("--long", type=int, default=2048, help="number of 512-token sequences")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--max-num-batched-tokens", type=int, default=32768)
    a = ap.parse_args()
    eng = EmbeddingEngine(a.model, device="cuda:0", max_num_batched_tokens=a.max_num_batched_tokens,
                          max_num_seqs=4096)
    res = [run(eng, a.short, 50, a.iters, a.warmup), run(eng, a.long, 512, a.iters, a.warmup)]
    ops.check_status()
    print(json.dumps({"metric": "embedding tokens/s/GPU", "model": a.model, "dtype": "bf16",
                      "data": "synthetic (uniform-random token ids, random-init weights)",
                      "results": res}))


if __name__ == "__main__":
    main()
