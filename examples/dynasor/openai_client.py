"""Chat with a reasoning model through the Dynasor proxy and print the early-exit statistics.

    python examples/dynasor/openai_client.py --base-url http://127.0.0.1:8000 --model MODEL \
        --probe-interval 32 --certainty-window 3 "What is 12 * 13?"
"""

import argparse
import json

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("question")
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="")
    ap.add_argument("--max-tokens", type=int, default=2048)
    ap.add_argument("--probe-interval", type=int, default=32)
    ap.add_argument("--certainty-window", type=int, default=3)
    ap.add_argument("--no-dynasor", action="store_true")
    a = ap.parse_args()
    body = {"model": a.model, "messages": [{"role": "user", "content": a.question}],
            "max_tokens": a.max_tokens, "stream": True}
    if not a.no_dynasor:
        body["dynasor"] = {"probe_interval": a.probe_interval, "certainty_window": a.certainty_window}
    with requests.post(a.base_url + "/v1/chat/completions", json=body, stream=True) as r:
        for line in r.iter_lines():
            if not line.startswith(b"data: ") or line == b"data: [DONE]":
                continue
            obj = json.loads(line[6:])
            if obj.get("object") == "dynasor.stats":
                print("\n[dynasor]", obj["dynasor"])
            for ch in obj.get("choices", []):
                print((ch.get("delta") or {}).get("content") or "", end="", flush=True)
    print()


if __name__ == "__main__":
    main()
