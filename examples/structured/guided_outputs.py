"""Structured outputs through the offline API: a choice, a regular expression and a JSON
schema, with suffix decoding on (drafts are cut to what the grammar allows).

    python examples/structured/guided_outputs.py [MODEL]
"""

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from arcticinference_b200 import LLM, SamplingParams  # noqa: E402

SCHEMA = {
    "type": "object",
    "required": ["title", "year"],
    "properties": {
        "title": {"type": "string", "maxLength": 60},
        "year": {"type": "integer"},
        "genres": {"type": "array", "items": {"enum": ["drama", "comedy", "sci-fi"]}, "maxItems": 3},
        "rating": {"type": ["number", "null"]},
    },
}


def main():
    model = sys.argv[1] if len(sys.argv) > 1 else "llama-tiny"
    llm = LLM(model=model, max_model_len=1024, speculative_config={"method": "suffix"})
    prompts = ["Is water wet? Answer yes or no.", "Give me a ticket number.",
               "Describe a film as JSON."]
    params = [SamplingParams(temperature=0.0, max_tokens=8, guided_choice=["yes", "no"]),
              SamplingParams(temperature=0.7, seed=1, max_tokens=16, guided_regex=r"TKT-\d{4}-[A-Z]{2}"),
              SamplingParams(temperature=0.7, seed=2, max_tokens=300, guided_json=SCHEMA)]
    for p, o in zip(prompts, llm.generate(prompts, params)):
        print(p, "->", o.outputs[0].text)
    print(json.loads(o.outputs[0].text))


if __name__ == "__main__":
    main()
