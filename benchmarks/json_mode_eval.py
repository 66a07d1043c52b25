"""JSON-mode evaluation: structured-output tasks answered under a JSON schema, scored on
whether every completion parses and conforms.

The reference's suite (tests/benchmarks/json_mode/task_description.py:6-33,
evaluate_text_json_mode.py) asks a served model to answer questions in the shape of small
pydantic models (a question with its answer, a rated answer, a list of facts, ...) through
the OpenAI API with guided JSON, and scores the answers' meaning with a sentence-embedding
model. This script keeps the task shapes and the guided-JSON transport and scores what can be
scored without that model: parse rate, schema conformance, tokens and time per document.

    python benchmarks/json_mode_eval.py --in-process llama-3.1-8b --num-questions 32
    python benchmarks/json_mode_eval.py --base-url http://127.0.0.1:8000 --model NAME
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

STR = lambda n=200: {"type": "string", "maxLength": n}                      # noqa: E731
TASKS = {
    "answer": {"type": "object", "properties": {"answer": STR()}},
    "answer_with_confidence": {"type": "object", "properties": {
        "answer": STR(), "confidence": {"type": "number"}}},
    "rated_answer": {"type": "object", "properties": {
        "answer": STR(), "rating": {"enum": [1, 2, 3, 4, 5]}, "is_factual": {"type": "boolean"}}},
    "facts": {"type": "object", "properties": {
        "topic": STR(60), "facts": {"type": "array", "items": STR(120), "minItems": 1,
                                    "maxItems": 4}}},
    "nested": {"type": "object", "properties": {
        "question": STR(), "parsed": {"type": "object", "properties": {
            "entities": {"type": "array", "items": STR(40), "maxItems": 5},
            "year": {"type": "integer"}}}}},
}
QUESTIONS = ["Who wrote the novel Dune?", "What is the capital of Australia?",
             "When did the Apollo 11 mission land on the Moon?", "What is the boiling point of water?",
             "Which planet has the most moons?", "Who painted the Mona Lisa?",
             "What is the largest ocean on Earth?", "What year did the Berlin Wall fall?"]


def conforms(schema: dict, text: str) -> bool:
    from arcticinference_b200.structured.json_schema import compile_schema
    return compile_schema(schema).validate(text)


def run_in_process(model: str, jobs: list, max_tokens: int, engine_kwargs: dict) -> list:
    from arcticinference_b200 import LLM, SamplingParams
    llm = LLM(model=model, **engine_kwargs)
    prompts = [p for p, _ in jobs]
    params = [SamplingParams(temperature=0.0, max_tokens=max_tokens, guided_json=s)
              for _, s in jobs]
    return [(o.outputs[0].text, len(o.outputs[0].token_ids)) for o in llm.generate(prompts, params)]


def run_http(base_url: str, model: str, jobs: list, max_tokens: int) -> list:
    import requests
    out = []
    for prompt, schema in jobs:
        r = requests.post(base_url.rstrip("/") + "/v1/chat/completions", timeout=600, json={
            "model": model, "max_tokens": max_tokens, "temperature": 0,
            "messages": [{"role": "user", "content": prompt}],
            "response_format": {"type": "json_schema", "json_schema": {"name": "t", "schema": schema}}})
        r.raise_for_status()
        body = r.json()
        out.append((body["choices"][0]["message"]["content"],
                    body.get("usage", {}).get("completion_tokens", 0)))
    return out


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--in-process", default=None, metavar="MODEL")
    ap.add_argument("--base-url", default=None)
    ap.add_argument("--model", default="")
    ap.add_argument("--num-questions", type=int, default=8)
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--engine-arg", action="append", default=[], metavar="K=V")
    a = ap.parse_args(argv)
    jobs = []
    for i in range(a.num_questions):
        q = QUESTIONS[i % len(QUESTIONS)]
        for name, schema in TASKS.items():
            jobs.append(("Answer as JSON (%s). %s" % (name, q), schema))
    t0 = time.perf_counter()
    if a.in_process:
        kw = {}
        for s in a.engine_arg:
            k, v = s.split("=", 1)
            try:
                v = json.loads(v)
            except json.JSONDecodeError:
                pass
            kw[k.replace("-", "_")] = v
        outs = run_in_process(a.in_process, jobs, a.max_tokens, kw)
    elif a.base_url:
        outs = run_http(a.base_url, a.model, jobs, a.max_tokens)
    else:
        ap.error("give --in-process MODEL or --base-url URL")
    wall = time.perf_counter() - t0
    parsed = ok = toks = 0
    for (text, n), (_, schema) in zip(outs, jobs):
        toks += n
        try:
            json.loads(text)
        except json.JSONDecodeError:
            continue
        parsed += 1
        ok += bool(conforms(schema, text))
    res = {"documents": len(jobs), "parse_rate": parsed / len(jobs), "conformance_rate": ok / len(jobs),
           "completion_tokens": toks, "seconds": wall, "documents_per_s": len(jobs) / wall}
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
