"""Early exit without the proxy: the client itself alternates generation chunks and probes
against any OpenAI-compatible completions endpoint (what the proxy automates).

    python examples/dynasor/naive_client.py --base-url http://127.0.0.1:8001 --model MODEL "question"
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import requests

from arcticinference_b200.dynasor.certainty import (DEFAULT_PROBE_SUFFIX, format_probe_prompt,
                                                    formalize_final_response, obtain_answer,
                                                    should_early_exit)


def complete(base, model, prompt, max_tokens, temperature):
    r = requests.post(base + "/v1/completions", json={"model": model, "prompt": prompt,
                                                      "max_tokens": max_tokens,
                                                      "temperature": temperature})
    r.raise_for_status()
    c = r.json()["choices"][0]
    return c["text"], c.get("finish_reason")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("question")
    ap.add_argument("--base-url", default="http://127.0.0.1:8001")
    ap.add_argument("--model", default="")
    ap.add_argument("--max-tokens", type=int, default=2048)
    ap.add_argument("--chunk", type=int, default=64, help="tokens generated between probes")
    ap.add_argument("--certainty-window", type=int, default=3)
    a = ap.parse_args()
    generated, answers, responses = "", [], []
    for _ in range(0, a.max_tokens, a.chunk):
        text, fr = complete(a.base_url, a.model, format_probe_prompt(a.question, generated, ""),
                            a.chunk, 0.7)
        generated += text
        print(text, end="", flush=True)
        if fr != "length" or not text:
            break
        probe, _ = complete(a.base_url, a.model,
                            format_probe_prompt(a.question, generated, DEFAULT_PROBE_SUFFIX), 32, 0.6)
        answers.append(obtain_answer(probe))
        responses.append(probe)
        if should_early_exit(answers, responses, a.certainty_window):
            print(formalize_final_response(generated, answers[-1]))
            break
    print()


if __name__ == "__main__":
    main()
