"""Chat through the offline API with an Arctic speculator (LSTM or MLP draft heads on the
target's hidden state) and suffix decoding side by side; the longer-scoring draft is verified
each step (reference example: projects/spec_dec/offline_inference_spec_dec.py:27-62).

    python examples/offline/spec_decode.py [MODEL] [SPECULATOR]

SPECULATOR is a speculator checkpoint directory; without one a randomly initialised LSTM
speculator of the right shape is attached (it drafts, and nearly every draft is rejected, so
the output equals plain decoding: the point is the plumbing).
"""

import sys

from _common import CONVERSATION, is_rank0, show

from arcticinference_b200 import LLM, SamplingParams  # noqa: E402


def main():
    model = sys.argv[1] if len(sys.argv) > 1 else "llama-3.1-8b"
    spec = {"method": "arctic", "num_speculative_tokens": 3, "enable_suffix_decoding": True,
            "disable_by_batch_size": 64}
    spec["model"] = sys.argv[2] if len(sys.argv) > 2 else "random"
    llm = LLM(model=model, quantization="fp8", speculative_config=spec, max_model_len=4096,
              seed=0)
    show(llm.chat(CONVERSATION, SamplingParams(temperature=0.1, max_tokens=128)))
    if is_rank0():
        st = llm.engine.get_stats()
        print("drafted per position:", st.get("drafted_per_position"))
        print("accepted per position:", st.get("accepted_per_position"))


if __name__ == "__main__":
    main()
