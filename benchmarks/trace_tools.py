"""Preparing and reading request traces for `trace_replay.py`.

    python benchmarks/trace_tools.py convert IN.csv OUT.jsonl [--from-min 0 --to-min 15]
    python benchmarks/trace_tools.py inspect TRACE.jsonl [--window-s 80] [--plot PREFIX]
    python benchmarks/trace_tools.py summarize REPLAY.csv [--plot PREFIX]

`convert` reads a public inference trace as CSV (columns ``TIMESTAMP`` as
``YYYY-mm-dd HH:MM:SS[.ffffff…]``, ``ContextTokens``, ``GeneratedTokens``) or a JSONL trace, keeps
the requests of a time window, re-bases the time stamps to milliseconds from the first kept
request and writes the replay schema ``{"timestamp", "input_length", "output_length"}``.
`inspect` prints what decides how hard a trace is to serve: requests that arrive together
(same time stamp) with their summed prompt lengths, the request rate per window, and the
length distributions. `summarize` reads the per-request CSV the replay writes
(``request,timestamp,input_len,output_len,ttft_ms,tpot_ms,e2el_ms``) and prints percentiles.
``--plot`` writes PNG files when matplotlib can be imported and says so when it cannot.

The reference prepares and plots traces with two scripts edited by hand
(benchmark/reproducibility/read_trace.py:7-71 for the parsing, :84-130 for the window and the
batch statistics; benchmark/reproducibility/plot.py for the TTFT / TPOT / latency plots).
"""

from __future__ import annotations

import argparse
import csv
import json
import sys
from collections import OrderedDict
from datetime import datetime
from typing import Optional

import numpy as np


def parse_timestamp(text: str) -> datetime:
    """``YYYY-mm-dd HH:MM:SS`` with any number of fractional digits (cut to microseconds)."""
    text = text.strip()
    if "." in text:
        whole, frac = text.split(".", 1)
        frac = "".join(ch for ch in frac if ch.isdigit())[:6]
        return datetime.strptime(whole + "." + (frac or "0"), "%Y-%m-%d %H:%M:%S.%f")
    return datetime.strptime(text, "%Y-%m-%d %H:%M:%S")


def read_records(path: str) -> list:
    """A trace as a list of ``{"timestamp": ms, "input_length", "output_length"}``; CSV time
    stamps become milliseconds from the file's first row."""
    recs = []
    if path.endswith(".csv"):
        with open(path, newline="") as f:
            rows = list(csv.DictReader(f))
        if not rows:
            return recs
        t0 = parse_timestamp(rows[0]["TIMESTAMP"])
        for r in rows:
            ms = (parse_timestamp(r["TIMESTAMP"]) - t0).total_seconds() * 1000.0
            recs.append({"timestamp": ms, "input_length": int(r["ContextTokens"]),
                         "output_length": int(r["GeneratedTokens"])})
        return recs
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            d = json.loads(line)
            recs.append({"timestamp": float(d["timestamp"]), "input_length": int(d["input_length"]),
                         "output_length": int(d["output_length"])})
    return recs


def window(recs: list, from_ms: float = 0.0, to_ms: Optional[float] = None,
           min_output: int = 1) -> list:
    """Requests with ``from_ms <= timestamp <= to_ms`` in time order, re-based to start at 0;
    requests that generate fewer than ``min_output`` tokens are dropped (a replay cannot time
    them)."""
    kept = [r for r in recs if r["timestamp"] >= from_ms and
            (to_ms is None or r["timestamp"] <= to_ms) and r["output_length"] >= min_output and
            r["input_length"] >= 1]
    kept.sort(key=lambda r: r["timestamp"])
    if not kept:
        return kept
    t0 = kept[0]["timestamp"]
    return [{"timestamp": int(round(r["timestamp"] - t0)), "input_length": r["input_length"],
             "output_length": r["output_length"]} for r in kept]


def write_jsonl(recs: list, path: str) -> None:
    with open(path, "w") as f:
        for r in recs:
            f.write(json.dumps(r) + "\n")


def arrival_groups(recs: list) -> "OrderedDict[int, tuple]":
    """time stamp (ms) -> (requests arriving then, their summed prompt length)."""
    groups: "OrderedDict[int, tuple]" = OrderedDict()
    for r in sorted(recs, key=lambda r: r["timestamp"]):
        ts = int(r["timestamp"])
        n, s = groups.get(ts, (0, 0))
        groups[ts] = (n + 1, s + r["input_length"])
    return groups


def request_rate(recs: list, window_s: float) -> list:
    """[(window start in s, requests per second)] over consecutive windows."""
    if not recs:
        return []
    ts = np.array([r["timestamp"] for r in recs], dtype=np.float64) / 1000.0
    edges = np.arange(0.0, ts.max() + window_s, window_s)
    if len(edges) < 2:
        edges = np.array([0.0, window_s])
    counts, _ = np.histogram(ts, bins=edges)
    return [(float(e), float(c) / window_s) for e, c in zip(edges[:-1], counts)]


def _pcts(x) -> dict:
    x = np.asarray(x, dtype=np.float64)
    if x.size == 0:
        return {}
    return {"mean": float(x.mean()), "p50": float(np.percentile(x, 50)),
            "p90": float(np.percentile(x, 90)), "p99": float(np.percentile(x, 99)),
            "max": float(x.max())}


def inspect(recs: list, window_s: float = 80.0) -> dict:
    groups = arrival_groups(recs)
    rate = request_rate(recs, window_s)
    span_s = (recs[-1]["timestamp"] - recs[0]["timestamp"]) / 1000.0 if len(recs) > 1 else 0.0
    return {
        "requests": len(recs), "span_s": span_s,
        "mean_rate_per_s": len(recs) / span_s if span_s > 0 else None,
        "peak_rate_per_s": max((r for _, r in rate), default=None),
        "arrival_groups": len(groups),
        "largest_group": max((n for n, _ in groups.values()), default=0),
        "largest_group_prompt_tokens": max((s for _, s in groups.values()), default=0),
        "input_length": _pcts([r["input_length"] for r in recs]),
        "output_length": _pcts([r["output_length"] for r in recs]),
        "total_input_tokens": int(sum(r["input_length"] for r in recs)),
        "total_output_tokens": int(sum(r["output_length"] for r in recs)),
    }


def read_replay_csv(path: str) -> list:
    rows = []
    with open(path, newline="") as f:
        for r in csv.DictReader(f):
            def num(k):
                v = r.get(k, "")
                return float(v) if v not in ("", "None", None) else None
            rows.append({"request": int(r["request"]), "timestamp": num("timestamp"),
                         "input_len": int(r["input_len"]), "output_len": int(r["output_len"]),
                         "ttft_ms": num("ttft_ms"), "tpot_ms": num("tpot_ms"),
                         "e2el_ms": num("e2el_ms")})
    return rows


def summarize(rows: list) -> dict:
    done = [r for r in rows if r["e2el_ms"] is not None]
    out = {"requests": len(rows), "completed": len(done)}
    for k in ("ttft_ms", "tpot_ms", "e2el_ms"):
        out[k] = _pcts([r[k] for r in done if r[k] is not None])
    if done:
        t_end = max(r["timestamp"] + r["e2el_ms"] for r in done)
        t_start = min(r["timestamp"] for r in done)
        dur = (t_end - t_start) / 1000.0
        toks = sum(r["input_len"] + r["output_len"] for r in done)
        out["duration_s"] = dur
        out["combined_tokens_per_s"] = toks / dur if dur > 0 else None
    return out


def _pyplot():
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        return plt
    except ImportError:
        print("matplotlib is not installed: no plots written", file=sys.stderr)
        return None


def plot_trace(recs: list, prefix: str, window_s: float) -> list:
    plt = _pyplot()
    if plt is None:
        return []
    files = []
    rate = request_rate(recs, window_s)
    series = [("rate", [t for t, _ in rate], [r for _, r in rate], "time (s)", "requests / s", "-"),
              ("output_length", list(range(len(recs))), [r["output_length"] for r in recs],
               "request", "output tokens", "-"),
              ("arrival", list(range(len(recs))), [r["timestamp"] / 1000.0 for r in recs],
               "request", "arrival (s)", "-")]
    for name, x, y, xl, yl, style in series:
        plt.figure(figsize=(10, 6))
        plt.plot(x, y, style)
        plt.xlabel(xl)
        plt.ylabel(yl)
        plt.grid(True)
        plt.tight_layout()
        files.append("%s_%s.png" % (prefix, name))
        plt.savefig(files[-1])
        plt.close()
    plt.figure(figsize=(10, 6))
    plt.scatter([r["output_length"] for r in recs], [r["input_length"] for r in recs], alpha=0.5)
    plt.xlabel("output tokens")
    plt.ylabel("prompt tokens")
    plt.yscale("log")
    plt.tight_layout()
    files.append("%s_lengths.png" % prefix)
    plt.savefig(files[-1])
    plt.close()
    return files


def plot_replay(rows: list, prefix: str) -> list:
    plt = _pyplot()
    if plt is None:
        return []
    files = []
    for key, style, log in (("ttft_ms", "-", False), ("tpot_ms", "o", True), ("e2el_ms", "o", False)):
        plt.figure()
        plt.plot([r[key] if r[key] is not None else float("nan") for r in rows], style)
        if log:
            plt.yscale("log")
        plt.xlabel("request")
        plt.ylabel("milliseconds")
        plt.title(key)
        files.append("%s_%s.png" % (prefix, key))
        plt.savefig(files[-1])
        plt.close()
    return files


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("convert")
    c.add_argument("src")
    c.add_argument("dst")
    c.add_argument("--from-min", type=float, default=0.0)
    c.add_argument("--to-min", type=float, default=None)
    c.add_argument("--limit", type=int, default=None)
    i = sub.add_parser("inspect")
    i.add_argument("trace")
    i.add_argument("--window-s", type=float, default=80.0)
    i.add_argument("--groups", action="store_true", help="list every arrival group")
    i.add_argument("--plot", default=None, metavar="PREFIX")
    s = sub.add_parser("summarize")
    s.add_argument("csv")
    s.add_argument("--plot", default=None, metavar="PREFIX")
    a = ap.parse_args(argv)

    if a.cmd == "convert":
        recs = window(read_records(a.src), a.from_min * 60e3,
                      None if a.to_min is None else a.to_min * 60e3)
        if a.limit:
            recs = recs[:a.limit]
        write_jsonl(recs, a.dst)
        res = {"written": len(recs), "path": a.dst}
    elif a.cmd == "inspect":
        recs = read_records(a.trace)
        res = inspect(recs, a.window_s)
        if a.groups:
            for ts, (n, toks) in arrival_groups(recs).items():
                print("%d ms: %d requests, %d prompt tokens" % (ts, n, toks))
        if a.plot:
            res["plots"] = plot_trace(recs, a.plot, a.window_s)
    else:
        rows = read_replay_csv(a.csv)
        res = summarize(rows)
        if a.plot:
            res["plots"] = plot_replay(rows, a.plot)
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
