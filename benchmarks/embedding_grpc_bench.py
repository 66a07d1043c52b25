"""Load generator for the embedding service (a replica or a replica manager) over gRPC.

Same workload as the reference's gRPC benchmark (benchmark/embedding/benchmark.py:118-121,
:210, :273-274): prompts are ``"hello " * (length - 4)``, the token count of a prompt is taken
as ``len(prompt.split()) + 2``, throughput is tokens over wall time, and batch sizes 1 / 16 /
64 are swept with ``--concurrency`` requests in flight. ``--token-ids`` sends pre-tokenised
int32 ids instead of text.

    python -m arcticinference_b200.embedding.replica_manager --model bert-base --num-replicas 8 &
    python benchmarks/embedding_grpc_bench.py --port 60050 --length 50 --batch-sizes 1,16,64
"""

import argparse
import asyncio
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from arcticinference_b200.embedding.client import InferenceClient  # noqa: E402


async def run_case(host, port, length, batch, n_requests, concurrency, token_ids, vocab):
    prompt = "hello " * max(length - 4, 1)
    tokens_per_prompt = len(prompt.split()) + 2
    rng = np.random.default_rng(0)
    sem = asyncio.Semaphore(concurrency)
    lat = []

    async with InferenceClient(host, port, timeout=600) as c:
        async def one():
            async with sem:
                t0 = time.perf_counter()
                if token_ids:
                    ids = [rng.integers(0, vocab, size=length).tolist() for _ in range(batch)]
                    out = await c.embed(token_ids=ids)
                else:
                    out = await c.embed(prompts=[prompt] * batch)
                assert out.shape[0] == batch
                lat.append(time.perf_counter() - t0)

        await asyncio.gather(*[one() for _ in range(min(4, n_requests))])     # warm-up
        lat.clear()
        t0 = time.perf_counter()
        await asyncio.gather(*[one() for _ in range(n_requests)])
        wall = time.perf_counter() - t0
    per = length if token_ids else tokens_per_prompt
    return {"length": length, "batch_size": batch, "requests": n_requests, "seconds": wall,
            "tokens_per_s": n_requests * batch * per / wall, "prompts_per_s": n_requests * batch / wall,
            "p50_latency_ms": float(np.percentile(lat, 50) * 1e3),
            "p99_latency_ms": float(np.percentile(lat, 99) * 1e3)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=60050)
    ap.add_argument("--length", type=int, default=50)
    ap.add_argument("--batch-sizes", default="1,16,64")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--token-ids", action="store_true")
    ap.add_argument("--vocab-size", type=int, default=30522)
    a = ap.parse_args()
    res = [asyncio.run(run_case(a.host, a.port, a.length, int(b), a.requests, a.concurrency,
                                a.token_ids, a.vocab_size)) for b in a.batch_sizes.split(",")]
    print(json.dumps({"metric": "embedding tokens/s (gRPC)", "results": res}))


if __name__ == "__main__":
    main()
