"""End-to-end serving suite: for each configuration start a real OpenAI-compatible server as
a subprocess, wait until it answers, run the performance tasks against it over HTTP, stop it,
and print one summary table.

Same shape as the reference's benchmark suite (tests/benchmarks/test_benchmarks.py with the
configurations of tests/benchmarks/benchmark_utils.py:22-116): configurations ``baseline``
(tensor parallel), ``shift`` (Ulysses + shift parallelism), ``swiftkv``, ``suffix``, ``spec``
(Arctic speculator), ``ulysses_spec`` and ``all``; tasks ``batch`` (random 2000-token prompts,
250 generated tokens, all sent at once: total token throughput), ``single`` (20 prompts at
concurrency 1: mean TTFT and TPOT) and ``json`` (guided-JSON documents: parse and conformance
rate). The accuracy tasks of the reference (lm_eval) need datasets and are not part of this
suite.

    python benchmarks/serving_suite.py --gpus 8 --model llama-3.1-8b --quantization fp8 \
        [--configs baseline,shift] [--tasks batch,single,json] [--num-prompts 2000]
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import subprocess
import sys
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "benchmarks"))

SPEC = {"method": "arctic", "model": "random", "num_speculative_tokens": 3,
        "disable_by_batch_size": 64}


def configurations(model: str, swiftkv_model: str, gpus: int) -> dict:
    """name -> (model, server flags, number of ranks)."""
    shift = ["--ulysses-sequence-parallel-size", str(gpus), "--enable-shift-parallel"] \
        if gpus > 1 else []
    tp = ["--tensor-parallel-size", str(gpus)] if gpus > 1 else []
    suffix = ["--speculative-config", json.dumps({"method": "suffix"})]
    spec = ["--speculative-config", json.dumps(SPEC)]
    hybrid = ["--speculative-config", json.dumps(dict(SPEC, enable_suffix_decoding=True))]
    return {
        "baseline": (model, tp, gpus),
        "shift": (model, shift, gpus),
        "swiftkv": (swiftkv_model, tp, gpus),
        "suffix": (model, tp + suffix, gpus),
        "spec": (model, tp + spec, gpus),
        "ulysses_spec": (model, shift + spec, gpus),
        "all": (swiftkv_model, shift + hybrid, gpus),
    }


class Server:
    """A ``serve`` subprocess (one process per GPU under torch.distributed.run when the
    configuration spans several ranks)."""

    def __init__(self, model: str, flags: list, ranks: int, port: int, common: list, log_path: str):
        serve = ["-m", "arcticinference_b200.cli", "serve", model, "--host", "127.0.0.1",
                 "--port", str(port), "--uvicorn-log-level", "warning"] + common + flags
        if ranks > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                   "--nproc-per-node", str(ranks), "--master-addr", "127.0.0.1",
                   "--master-port", str(port + 1000)] + serve
        else:
            cmd = [sys.executable] + serve
        self.url = "http://127.0.0.1:%d" % port
        self.log = open(log_path, "w")
        env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        self.proc = subprocess.Popen(cmd, stdout=self.log, stderr=subprocess.STDOUT, env=env,
                                     cwd=ROOT, start_new_session=True)

    def wait_ready(self, timeout: float) -> None:
        deadline = time.time() + timeout
        while time.time() < deadline:
            if self.proc.poll() is not None:
                raise RuntimeError("server exited with code %s (see its log)" % self.proc.returncode)
            try:
                with urllib.request.urlopen(self.url + "/v1/models", timeout=2) as r:
                    if r.status == 200:
                        return
            except OSError:
                time.sleep(0.5)
        raise TimeoutError("server did not answer within %d s" % timeout)

    def stop(self) -> None:
        import signal
        if self.proc.poll() is None:
            try:
                os.killpg(self.proc.pid, signal.SIGTERM)      # the group this class started
            except ProcessLookupError:
                pass
            try:
                self.proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                os.killpg(self.proc.pid, signal.SIGKILL)
                self.proc.wait(timeout=10)
        self.log.close()


# ------------------------------------------------------------------------------- tasks
def task_batch(url, model, vocab, a) -> dict:
    import trace_replay as tr
    reqs = [tr.TraceRequest(i, 0.0, a.input_len, a.output_len) for i in range(a.num_prompts)]
    res = asyncio.run(tr.replay(tr.HttpTarget(url, model, vocab), reqs))
    return {"total_token_throughput": res["combined_tokens_per_s"], "completed": res["completed"],
            "failed": res["failed"], "p50_ttft_ms": res["p50_ttft_ms"], "p50_tpot_ms": res["p50_tpot_ms"]}


def task_single(url, model, vocab, a) -> dict:
    import numpy as np
    import trace_replay as tr

    async def run():
        target = tr.HttpTarget(url, model, vocab)
        rng = np.random.default_rng(1)
        reqs = [tr.TraceRequest(i, 0.0, a.input_len, a.output_len) for i in range(a.single_prompts)]
        for r in reqs:                       # one request in flight
            await target.run(r, rng.integers(0, vocab, size=r.input_len).tolist())
        await target.aclose()
        return reqs
    reqs = asyncio.run(run())
    ttft = [r.ttft_ms for r in reqs if r.ttft_ms is not None]
    tpot = [r.tpot_ms for r in reqs if r.tpot_ms is not None]
    mean = lambda xs: sum(xs) / len(xs) if xs else None          # noqa: E731
    return {"mean_ttft_ms": mean(ttft), "mean_tpot_ms": mean(tpot),
            "failed": sum(r.error is not None for r in reqs)}


def task_json(url, model, vocab, a) -> dict:
    import json_mode_eval as jm
    res = jm.main(["--base-url", url, "--model", model, "--num-questions", str(a.json_questions),
                   "--max-tokens", str(a.json_max_tokens)])
    return {"parse_rate": res["parse_rate"], "conformance_rate": res["conformance_rate"],
            "documents_per_s": res["documents_per_s"]}


TASKS = {"batch": task_batch, "single": task_single, "json": task_json}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--swiftkv-model", default=None, help="default: MODEL-swiftkv")
    ap.add_argument("--quantization", default="fp8")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--configs", default="baseline,shift,swiftkv,suffix,spec,ulysses_spec,all")
    ap.add_argument("--tasks", default="batch,single")
    ap.add_argument("--num-prompts", type=int, default=2000)
    ap.add_argument("--single-prompts", type=int, default=20)
    ap.add_argument("--input-len", type=int, default=2000)
    ap.add_argument("--output-len", type=int, default=250)
    ap.add_argument("--json-questions", type=int, default=8)
    ap.add_argument("--json-max-tokens", type=int, default=512)
    ap.add_argument("--vocab-size", type=int, default=128256)
    ap.add_argument("--port", type=int, default=18000)
    ap.add_argument("--ready-timeout", type=float, default=900)
    ap.add_argument("--device", default=None)
    ap.add_argument("--log-dir", default=".")
    ap.add_argument("--server-arg", action="append", default=[], metavar="FLAG",
                    help="extra flag for every server, e.g. --server-arg=--max-model-len=4096")
    a = ap.parse_args(argv)
    swift = a.swiftkv_model or a.model + "-swiftkv"
    common = ["--max-model-len", str(a.input_len + a.output_len + 64), "--no-enable-prefix-caching"]
    if str(a.quantization).lower() not in ("none", "bf16", ""):
        common += ["--quantization", a.quantization]
    if a.device:
        common += ["--device", a.device]
    for extra in a.server_arg:
        common += extra.split("=", 1) if extra.startswith("--") and "=" in extra else [extra]
    table = configurations(a.model, swift, a.gpus)
    results: dict = {}
    for i, name in enumerate(c for c in a.configs.split(",") if c):
        if name not in table:
            ap.error("unknown configuration %r" % name)
        model, flags, ranks = table[name]
        srv = Server(model, flags, ranks, a.port + i, common,
                     os.path.join(a.log_dir, "serving_suite_%s.log" % name))
        row: dict = {}
        try:
            srv.wait_ready(a.ready_timeout)
            for task in (t for t in a.tasks.split(",") if t):
                row[task] = TASKS[task](srv.url, model, a.vocab_size, a)
        except Exception as e:  # noqa: BLE001 - a failed configuration is a row of the table
            row["error"] = "%s: %s" % (type(e).__name__, e)
        finally:
            srv.stop()
        results[name] = row
        print(json.dumps({"config": name, **row}), flush=True)
    # summary table
    cols = [("batch", "total_token_throughput", "tok/s"), ("single", "mean_ttft_ms", "TTFT ms"),
            ("single", "mean_tpot_ms", "TPOT ms"), ("json", "conformance_rate", "JSON ok")]
    print("%-14s" % "config" + "".join("%14s" % c[2] for c in cols))
    for name, row in results.items():
        cells = []
        for task, key, _ in cols:
            v = row.get(task, {}).get(key)
            cells.append("%14s" % ("-" if v is None else "%.1f" % v if v >= 10 else "%.3f" % v))
        print("%-14s" % name + "".join(cells) + ("   " + row["error"] if "error" in row else ""))
    return results


if __name__ == "__main__":
    main()
