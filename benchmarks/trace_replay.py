"""Open-loop trace replay: request i is sent at ``timestamp_i`` whatever the server's state,
with a random prompt of ``input_length`` tokens and a forced ``output_length`` (EOS ignored).
Reports per-request TTFT / TPOT / end-to-end latency and aggregate throughput.

Trace: JSONL, one request per line, ``{"timestamp": ms, "input_length": n, "output_length": m}``
(the schema of the reference's replay patch: benchmark/reproducibility/patches_v0.10.1/
serve.py:101-116, datasets.py:353-373). ``--synthetic N`` generates one instead: Poisson
arrivals at ``--rate`` requests/s, log-normal prompt lengths, fixed output length.

Targets:
    --base-url http://host:port     an OpenAI-compatible server (streaming completions);
                                    several, comma-separated: least requests in flight
    --in-process MODEL [--engine-arg k=v ...]   an engine inside this process

    python benchmarks/trace_replay.py --in-process llama-3.1-8b --synthetic 256 --rate 8 \
        --csv out.csv
"""

from __future__ import annotations

import argparse
import asyncio
import csv
import json
import math
import os
import sys
import time
from dataclasses import dataclass
from typing import Optional

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@dataclass
class TraceRequest:
    index: int
    timestamp_ms: float
    input_len: int
    output_len: int
    ttft_ms: Optional[float] = None
    tpot_ms: Optional[float] = None
    e2el_ms: Optional[float] = None
    generated: int = 0
    error: Optional[str] = None


def load_trace(path: str, limit: Optional[int] = None) -> list:
    out = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            d = json.loads(line)
            out.append(TraceRequest(len(out), float(d["timestamp"]), int(d["input_length"]),
                                    int(d["output_length"])))
            if limit and len(out) >= limit:
                break
    t0 = min(r.timestamp_ms for r in out) if out else 0.0
    for r in out:
        r.timestamp_ms -= t0
    return sorted(out, key=lambda r: r.timestamp_ms)


def synthetic_trace(n: int, rate: float, median_in: int = 2000, sigma: float = 1.0,
                    min_in: int = 1, max_in: int = 32768, output_len: int = 256, seed: int = 0) -> list:
    rng = np.random.default_rng(seed)
    t = np.cumsum(rng.exponential(1.0 / rate, size=n)) * 1e3
    lens = np.clip(np.exp(rng.normal(math.log(median_in), sigma, size=n)), min_in, max_in).astype(int)
    return [TraceRequest(i, float(t[i] - t[0]), int(lens[i]), output_len) for i in range(n)]


def save_trace(reqs: list, path: str) -> None:
    with open(path, "w") as f:
        for r in reqs:
            f.write(json.dumps({"timestamp": r.timestamp_ms, "input_length": r.input_len,
                                "output_length": r.output_len}) + "\n")


# ------------------------------------------------------------------------------ targets
class InProcessTarget:
    def __init__(self, model: str, engine_kwargs: dict):
        from arcticinference_b200.config import EngineArgs
        from arcticinference_b200.engine.async_llm import AsyncLLM
        self.llm = AsyncLLM.from_engine_args(EngineArgs(model=model, **engine_kwargs)).start()
        self.vocab = self.llm.engine.config.model.vocab_size

    async def run(self, req: TraceRequest, prompt: list) -> None:
        from arcticinference_b200.engine.sampling_params import SamplingParams
        sp = SamplingParams(temperature=0.0, max_tokens=req.output_len, ignore_eos=True)
        t0 = time.perf_counter()
        first = None
        n = 0
        async for out in self.llm.generate(prompt, sp, "trace-%d" % req.index):
            n = len(out.outputs[0].token_ids)
            if first is None and n > 0:
                first = time.perf_counter()
        t1 = time.perf_counter()
        finish(req, t0, first, t1, n)

    def close(self) -> None:
        self.llm.shutdown()


class HttpTarget:
    """An OpenAI-compatible server, or several behind a comma-separated ``base_url``: each
    request then goes to the server with the fewest requests of this client in flight (the
    independent-replicas layout of a parallelism comparison)."""

    def __init__(self, base_url: str, model: str, vocab: int):
        import aiohttp
        self.bases = [u.strip().rstrip("/") for u in base_url.split(",") if u.strip()]
        self.inflight = [0] * len(self.bases)
        self.sent = [0] * len(self.bases)
        self.model = model
        self.vocab = vocab
        self.session = None
        self._aiohttp = aiohttp

    async def run(self, req: TraceRequest, prompt: list) -> None:
        if self.session is None:
            self.session = self._aiohttp.ClientSession(
                timeout=self._aiohttp.ClientTimeout(total=None))
        body = {"model": self.model, "prompt": prompt, "max_tokens": req.output_len,
                "temperature": 0.0, "ignore_eos": True, "stream": True}
        which = min(range(len(self.bases)), key=lambda i: (self.inflight[i], self.sent[i]))
        self.inflight[which] += 1
        self.sent[which] += 1
        t0 = time.perf_counter()
        first = None
        n = 0
        try:
            async with self.session.post(self.bases[which] + "/v1/completions", json=body) as resp:
                if resp.status != 200:
                    req.error = "HTTP %d" % resp.status
                    return
                async for raw in resp.content:
                    if not raw.startswith(b"data: {"):
                        continue
                    obj = json.loads(raw[6:])
                    if obj.get("usage"):
                        n = obj["usage"]["completion_tokens"]
                    if first is None and any(c.get("text") for c in obj.get("choices", [])):
                        first = time.perf_counter()
        finally:
            self.inflight[which] -= 1
        finish(req, t0, first, time.perf_counter(), n or req.output_len)

    def close(self) -> None:
        pass

    async def aclose(self) -> None:
        if self.session is not None:
            await self.session.close()


def finish(req: TraceRequest, t0: float, first: Optional[float], t1: float, n: int) -> None:
    req.generated = n
    req.e2el_ms = (t1 - t0) * 1e3
    if first is not None:
        req.ttft_ms = (first - t0) * 1e3
        if n > 1:
            req.tpot_ms = (t1 - first) * 1e3 / (n - 1)


# ------------------------------------------------------------------------------ replay
async def replay(target, reqs: list, speed: float = 1.0, seed: int = 0) -> dict:
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, target.vocab, size=r.input_len).tolist() for r in reqs]
    start = time.perf_counter()

    async def one(r: TraceRequest, p: list) -> None:
        delay = r.timestamp_ms / 1e3 / speed - (time.perf_counter() - start)
        if delay > 0:
            await asyncio.sleep(delay)
        try:
            await target.run(r, p)
        except Exception as e:  # noqa: BLE001 - recorded per request
            r.error = "%s: %s" % (type(e).__name__, e)

    await asyncio.gather(*[one(r, p) for r, p in zip(reqs, prompts)])
    wall = time.perf_counter() - start
    if hasattr(target, "aclose"):
        await target.aclose()
    return summarize(reqs, wall)


def summarize(reqs: list, wall: float) -> dict:
    ok = [r for r in reqs if r.error is None and r.e2el_ms is not None]
    pct = lambda xs, q: float(np.percentile(xs, q)) if len(xs) else None
    ttft = [r.ttft_ms for r in ok if r.ttft_ms is not None]
    tpot = [r.tpot_ms for r in ok if r.tpot_ms is not None]
    e2e = [r.e2el_ms for r in ok]
    tin, tout = sum(r.input_len for r in ok), sum(r.generated for r in ok)
    return {"requests": len(reqs), "completed": len(ok), "failed": len(reqs) - len(ok),
            "duration_s": wall, "input_tokens": tin, "output_tokens": tout,
            "combined_tokens_per_s": (tin + tout) / wall if wall > 0 else 0.0,
            "output_tokens_per_s": tout / wall if wall > 0 else 0.0,
            "request_throughput": len(ok) / wall if wall > 0 else 0.0,
            "p50_ttft_ms": pct(ttft, 50), "p99_ttft_ms": pct(ttft, 99),
            "p50_tpot_ms": pct(tpot, 50), "p99_tpot_ms": pct(tpot, 99),
            "p50_e2el_ms": pct(e2e, 50), "p99_e2el_ms": pct(e2e, 99)}


def write_csv(reqs: list, path: str) -> None:
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["request", "timestamp", "input_len", "output_len", "ttft_ms", "tpot_ms", "e2el_ms"])
        for r in reqs:
            w.writerow([r.index, r.timestamp_ms, r.input_len, r.output_len, r.ttft_ms, r.tpot_ms,
                        r.e2el_ms])


def _kv(s: str):
    k, v = s.split("=", 1)
    try:
        v = json.loads(v)
    except json.JSONDecodeError:
        pass
    return k.replace("-", "_"), v


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--trace-dataset-path", "--trace", dest="trace", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--rate", type=float, default=8.0)
    ap.add_argument("--median-input", type=int, default=2000)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--max-input", type=int, default=32768)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--limit", type=int, default=None)
    ap.add_argument("--speed", type=float, default=1.0, help="replay speed-up factor")
    ap.add_argument("--base-url", default=None)
    ap.add_argument("--model", default="")
    ap.add_argument("--vocab-size", type=int, default=128256)
    ap.add_argument("--in-process", default=None, metavar="MODEL")
    ap.add_argument("--engine-arg", action="append", default=[], metavar="K=V")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--save-trace", default=None)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.trace:
        reqs = load_trace(a.trace, a.limit)
    elif a.synthetic:
        reqs = synthetic_trace(a.synthetic, a.rate, a.median_input, a.sigma, 1, a.max_input,
                               a.output_len, a.seed)
    else:
        ap.error("give --trace-dataset-path or --synthetic N")
    if a.save_trace:
        save_trace(reqs, a.save_trace)
    if a.in_process:
        target = InProcessTarget(a.in_process, dict(_kv(s) for s in a.engine_arg))
    elif a.base_url:
        target = HttpTarget(a.base_url, a.model, a.vocab_size)
    else:
        ap.error("give --base-url or --in-process")
    try:
        res = asyncio.run(replay(target, reqs, a.speed, a.seed))
    finally:
        target.close()
    if a.csv:
        write_csv(reqs, a.csv)
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
