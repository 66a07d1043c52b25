"""A dataset job on a replica pool: bounded concurrency, retries, results in dataset order.

    python examples/server/pipeline_example.py [--fake]
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import asyncio

from arcticinference_b200.server.config import ServerModelConfig
from arcticinference_b200.server.pipeline import Pipeline
from arcticinference_b200.server.replica_pool import ReplicaPool


async def main(fake: bool):
    kw = {}
    if fake:
        from arcticinference_b200.server.testing import DummyWorker
        kw = dict(worker_factory=lambda i: DummyWorker(i), gpu_ids=list(range(4)))
    pool = ReplicaPool(**kw)
    await pool.initialize(ServerModelConfig(model="llama-3.1-8b", quantization="fp8"))
    pipe = Pipeline(pool)

    @pipe.task(max_in_flight=256, retries=2)
    async def summarize(item, generate):
        out = await generate("Summarize: " + item["text"], {"max_tokens": 64, "temperature": 0.0},
                             routing_key=item["doc"])          # same document -> same replica
        return {"doc": item["doc"], "summary": out["text"]}

    data = [{"doc": "d%d" % (i % 10), "text": "paragraph %d" % i} for i in range(100)]
    res = await summarize.run(data, progress=lambda done, n: None)
    print(len(res), "results;", res[0])

    # the same job in the reference's call shape: one registered task, run by the pipeline,
    # sampling parameters as keywords, text returned
    @pipe.task
    async def title(sample, llm):
        return await llm.generate(prompt="Title for: " + sample["text"], max_tokens=8, temperature=0.0)

    titles = await pipe.run(data[:10], max_retries=2)
    print(len(titles), "titles;", titles[0])
    await pool.shutdown()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--fake", action="store_true")
    asyncio.run(main(ap.parse_args().fake))
