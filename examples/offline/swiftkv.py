"""Chat through the offline API with a SwiftKV model: prompt tokens run only the first
``num_key_value_layers`` layers, the later layers' K/V come from one projection of that
boundary's hidden state, and only the sampled positions go through the later layers
(reference example: projects/swiftkv/offline_inference_swiftkv.py:21-44).

    python examples/offline/swiftkv.py [MODEL]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/offline/swiftkv.py [MODEL]          # tensor parallel over 2 GPUs

MODEL is a SwiftKV checkpoint directory (``model_type: llama_swiftkv``) or the built-in
``llama-3.1-8b-swiftkv`` architecture with random weights.
"""

import os
import sys

from _common import CONVERSATION, show

from arcticinference_b200 import LLM, SamplingParams  # noqa: E402


def main():
    model = sys.argv[1] if len(sys.argv) > 1 else "llama-3.1-8b-swiftkv"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    llm = LLM(model=model, tensor_parallel_size=world, max_model_len=8192)
    show(llm.chat(CONVERSATION, SamplingParams(temperature=0.1, max_tokens=800)))


if __name__ == "__main__":
    main()
