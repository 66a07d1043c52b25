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
                       "--output-len", "4", "--model", "tiny",
                       # two "replicas" (the same server under two spellings): least in flight
                       "--base-url", "http://127.0.0.1:18441, http://localhost:18441/",
                       "--vocab-size", "1000"])
        assert res["completed"] == 4 and res["output_tokens"] == 16 and res["p50_ttft_ms"] > 0
    finally:
        srv.should_exit = True
        th.join(5)
        llm.shutdown()


def test_trace_tools_convert_inspect_summarize(tmp_path):
    import trace_tools as tt
    src = tmp_path / "t.csv"
    with open(src, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["TIMESTAMP", "ContextTokens", "GeneratedTokens"])
        w.writerow(["2023-11-16 18:15:46.6805900", 374, 44])       # 7 fractional digits
        w.writerow(["2023-11-16 18:15:50.9951690", 396, 109])
        w.writerow(["2023-11-16 18:15:50.9951690", 879, 55])       # arrives with the one before
        w.writerow(["2023-11-16 18:16:51", 1000, 0])               # generates nothing: dropped
        w.writerow(["2023-11-16 18:17:46.680590", 91, 7])          # exactly 2 minutes in
        w.writerow(["2023-11-16 18:30:00.0", 5, 5])                # outside the window
    assert tt.parse_timestamp("2023-11-16 18:15:46.6805900").microsecond == 680590
    dst = tmp_path / "t.jsonl"
    res = tt.main(["convert", str(src), str(dst), "--from-min", "0.05", "--to-min", "2"])
    assert res["written"] == 3
    recs = tt.read_records(str(dst))
    # re-based to the first kept request (the 4.3 s one)
    assert [r["timestamp"] for r in recs] == [0.0, 0.0, 115685.0]
    assert [r["input_length"] for r in recs] == [396, 879, 91]
    assert tr.load_trace(str(dst))[2].output_len == 7              # the replay reads it

    info = tt.main(["inspect", str(dst), "--window-s", "60", "--groups"])
    assert info["requests"] == 3 and info["arrival_groups"] == 2
    assert info["largest_group"] == 2 and info["largest_group_prompt_tokens"] == 396 + 879
    assert info["total_output_tokens"] == 109 + 55 + 7
    assert info["peak_rate_per_s"] == pytest.approx(2 / 60)
    assert tt.request_rate(recs, 60.0) == [(0.0, pytest.approx(2 / 60)), (60.0, pytest.approx(1 / 60))]

    rep = tmp_path / "r.csv"
    reqs = [tr.TraceRequest(0, 0.0, 10, 5, 20.0, 2.0, 28.0), tr.TraceRequest(1, 100.0, 30, 5, 40.0, 4.0, 56.0),
            tr.TraceRequest(2, 200.0, 30, 5)]                      # one that failed
    tr.write_csv(reqs, str(rep))
    summ = tt.main(["summarize", str(rep)])
    assert summ["requests"] == 3 and summ["completed"] == 2
    assert summ["ttft_ms"]["p50"] == pytest.approx(30.0) and summ["tpot_ms"]["max"] == 4.0
    assert summ["duration_s"] == pytest.approx(0.156)
    assert summ["combined_tokens_per_s"] == pytest.approx(50 / 0.156)
