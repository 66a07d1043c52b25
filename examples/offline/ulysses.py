"""Chat through the offline API with Ulysses sequence parallelism and shift parallelism: long
prompts are split over the ranks by tokens, small decode batches run tensor-parallel over the
same ranks on the same KV cache (reference example: projects/ulysses/
offline_inference_ulysses.py:23-50).

One process per GPU:

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 \
        examples/offline/ulysses.py [MODEL]

MODEL is a checkpoint directory or one of the built-in architectures (random weights), e.g.
``llama-3.1-8b``.
"""

import os
import sys

from _common import CONVERSATION, show

from arcticinference_b200 import LLM, SamplingParams  # noqa: E402


def main():
    model = sys.argv[1] if len(sys.argv) > 1 else "llama-3.1-8b"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    llm = LLM(model=model, quantization="fp8", tensor_parallel_size=1,
              ulysses_sequence_parallel_size=world, enable_shift_parallel=world > 1,
              max_model_len=8192)
    show(llm.chat(CONVERSATION, SamplingParams(temperature=0.1, max_tokens=800)))


if __name__ == "__main__":
    main()
