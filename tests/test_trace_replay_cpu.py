"""Trace replay client: trace IO, the synthetic generator, and a replay against an in-process
CPU engine and against the OpenAI-compatible server."""

import csv
import json
import os
import sys
import threading
import time

import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))
import trace_replay as tr  # noqa: E402


def test_trace_io_and_synthetic(tmp_path):
    reqs = tr.synthetic_trace(200, rate=8.0, median_in=2000, sigma=1.0, max_in=32768, output_len=256, seed=0)
    gaps = [b.timestamp_ms - a.timestamp_ms for a, b in zip(reqs, reqs[1:])]
    assert 90 < sum(gaps) / len(gaps) < 170                       # 8 req/s -> 125 ms mean gap
    lens = sorted(r.input_len for r in reqs)
    assert 1200 < lens[100] < 3200 and lens[0] >= 1 and lens[-1] <= 32768
    p = tmp_path / "t.jsonl"
    tr.save_trace(reqs, str(p))
    back = tr.load_trace(str(p), limit=50)
    assert len(back) == 50 and back[0].timestamp_ms == 0.0 and back[7].input_len == reqs[7].input_len
    ex = tr.load_trace(os.path.join(os.path.dirname(tr.__file__), "example_trace.jsonl"))
    assert len(ex) == 32 and all(r.output_len > 0 for r in ex)


def test_replay_in_process(tmp_path):
    out = tmp_path / "r.csv"
    res = tr.main(["--synthetic", "6", "--rate", "50", "--median-input", "20", "--sigma", "0.3",
                   "--max-input", "60", "--output-len", "5", "--in-process", "llama-tiny",
                   "--engine-arg", "max_model_len=128", "--engine-arg", "num_gpu_blocks_override=64",
                   "--engine-arg", "block_size=16", "--csv", str(out)])
    assert res["completed"] == 6 and res["failed"] == 0 and res["output_tokens"] == 30
    assert res["p50_ttft_ms"] > 0 and res["p50_tpot_ms"] > 0 and res["combined_tokens_per_s"] > 0
    rows = list(csv.reader(open(out)))
    assert rows[0] == ["request", "timestamp", "input_len", "output_len", "ttft_ms", "tpot_ms", "e2el_ms"]
    assert len(rows) == 7 and float(rows[1][6]) > 0


def test_replay_over_http():
    import uvicorn
    from arcticinference_b200.config import EngineArgs
    from arcticinference_b200.engine.async_llm import AsyncLLM
    from arcticinference_b200.entrypoints.openai_server import build_app
    llm = AsyncLLM.from_engine_args(EngineArgs(model="llama-tiny", max_model_len=128, block_size=16,
                                               num_gpu_blocks_override=64), device="cpu").start()
    srv = uvicorn.Server(uvicorn.Config(build_app(llm, "tiny"), host="127.0.0.1", port=18441,
                                        log_level="warning"))
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    for _ in range(200):
        if srv.started:
            break
        time.sleep(0.05)
    try:
        res = tr.main(["--synthetic", "4", "--rate", "100", "--median-input", "10", "--sigma", "0.1",
                       "--output-len", "4", "--base-url", "http://127.0.0.1:18441", "--model", "tiny",
                       "--vocab-size", "1000"])
        assert res["completed"] == 4 and res["output_tokens"] == 16 and res["p50_ttft_ms"] > 0
    finally:
        srv.should_exit = True
        th.join(5)
        llm.shutdown()
