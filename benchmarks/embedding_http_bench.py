"""Load generator for an OpenAI-compatible ``/v1/embeddings`` endpoint (this package's
``python -m arcticinference_b200.embedding.http_server`` or any other server).

Counterpart of the gRPC generator beside it, with the reference's workload definition
(benchmark/embedding/benchmark_http.py; prompts ``"hello " * (length - 4)``, token count
``len(prompt.split()) + 2`` per prompt, throughput = tokens / wall time). ``--token-ids``
sends random pre-tokenised ids of exactly ``--length`` tokens instead of text.

    python -m arcticinference_b200.embedding.http_server --model bert-base --port 8000 &
    python benchmarks/embedding_http_bench.py --base-url http://127.0.0.1:8000 --length 50 \
        --batch-sizes 1,16,64
"""

import argparse
import asyncio
import base64
import json
import time

import numpy as np


async def run_case(base_url, model, length, batch, n_requests, concurrency, token_ids, vocab,
                   encoding_format="base64"):
    import aiohttp
    prompt = "hello " * max(length - 4, 1)
    tokens_per_prompt = len(prompt.split()) + 2
    rng = np.random.default_rng(0)
    sem = asyncio.Semaphore(concurrency)
    lat = []
    url = base_url.rstrip("/") + "/v1/embeddings"
    timeout = aiohttp.ClientTimeout(total=600)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def one():
            async with sem:
                if token_ids:
                    inp = [rng.integers(0, vocab, size=length).tolist() for _ in range(batch)]
                else:
                    inp = [prompt] * batch
                t0 = time.perf_counter()
                async with session.post(url, json={"model": model, "input": inp,
                                                   "encoding_format": encoding_format}) as r:
                    if r.status != 200:
                        raise RuntimeError("HTTP %d: %s" % (r.status, await r.text()))
                    body = await r.json()
                assert len(body["data"]) == batch
                if encoding_format == "base64":
                    v = np.frombuffer(base64.b64decode(body["data"][0]["embedding"]), dtype="<f4")
                    assert v.size > 0
                lat.append(time.perf_counter() - t0)

        await asyncio.gather(*[one() for _ in range(min(4, n_requests))])     # warm-up
        lat.clear()
        t0 = time.perf_counter()
        await asyncio.gather(*[one() for _ in range(n_requests)])
        wall = time.perf_counter() - t0
    per = length if token_ids else tokens_per_prompt
    return {"length": length, "batch_size": batch, "requests": n_requests, "seconds": wall,
            "tokens_per_s": n_requests * batch * per / wall,
            "prompts_per_s": n_requests * batch / wall,
            "p50_latency_ms": float(np.percentile(lat, 50) * 1e3),
            "p99_latency_ms": float(np.percentile(lat, 99) * 1e3)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="bert-base")
    ap.add_argument("--length", type=int, default=50)
    ap.add_argument("--batch-sizes", default="1,16,64")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--concurrency", type=int, default=32)
    ap.add_argument("--token-ids", action="store_true")
    ap.add_argument("--vocab-size", type=int, default=30522)
    ap.add_argument("--encoding-format", default="base64", choices=["base64", "float"])
    a = ap.parse_args(argv)
    out = []
    for b in [int(x) for x in a.batch_sizes.split(",")]:
        r = asyncio.run(run_case(a.base_url, a.model, a.length, b, a.requests, a.concurrency,
                                 a.token_ids, a.vocab_size, a.encoding_format))
        print(json.dumps(r))
        out.append(r)
    return out


if __name__ == "__main__":
    main()
