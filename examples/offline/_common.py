"""Shared bits of the offline examples: the conversation and the rank-0 print."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

CONVERSATION = [
    {"role": "user", "content": "Hello"},
    {"role": "assistant", "content": "Hello! How can I assist you today?"},
    {"role": "user", "content": "Write an essay about the importance of higher education."},
]


def is_rank0() -> bool:
    return int(os.environ.get("RANK", "0")) == 0


def show(outputs) -> None:
    if is_rank0():
        print("=" * 80)
        out = outputs[0].outputs[0]
        print(out.text)
        print("-" * 80)
        print("%d prompt tokens, %d generated, finish reason %s"
              % (len(outputs[0].prompt_token_ids), len(out.token_ids), out.finish_reason))
