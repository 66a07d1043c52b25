"""Two models on one machine through the multi-model driver: GPUs are shared evenly, the
first model shrinks when the second arrives and grows back when it leaves.

    python examples/server/driver_example.py [--fake]      # --fake: CPU stand-in workers
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import asyncio

from arcticinference_b200.server.config import ServerModelConfig
from arcticinference_b200.server.multi_model import Driver


async def main(fake: bool):
    kw = {}
    if fake:
        from arcticinference_b200.server.testing import DummyWorker
        kw = dict(worker_factory=lambda i: DummyWorker(i), gpu_ids=list(range(8)))
    d = Driver(**kw)
    a = ServerModelConfig(model="llama-3.1-8b", quantization="fp8", max_model_len=8192)
    b = ServerModelConfig(model="llama-3.1-8b-swiftkv", quantization="fp8", max_model_len=8192,
                          ulysses_sequence_parallel_size=2, enable_shift_parallel=True)
    print("model a replicas:", await d.initialize(a, model_id="a"))
    print("model b replicas:", await d.initialize(b, model_id="b"))
    print((await d.get_status())["models"]["a"]["num_replicas"], "replicas of a after rebalancing")
    outs = await d.generate(["Hello", [1, 2, 3]], {"max_tokens": 8}, model_id="b")
    print([o["generation_len"] for o in outs])
    await d.shutdown("b")
    await d.wait_scaling()
    print((await d.get_status())["models"]["a"]["num_replicas"], "replicas of a after b left")
    await d.shutdown()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--fake", action="store_true")
    asyncio.run(main(ap.parse_args().fake))
