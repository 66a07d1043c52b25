"""The benchmark scripts run end to end on the CPU path with a tiny model."""

import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "benchmarks", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_latency_bench_reports_ttft_and_tpot():
    res = _load("latency_bench").main(["--model", "llama-tiny", "--quantization", "none",
                                       "--num-prompts", "2", "--warmup", "1", "--input-len", "30",
                                       "--output-len", "6", "--device", "cpu"])
    assert res["task"] == "single" and res["num_prompts"] == 2
    assert res["mean_ttft_ms"] > 0 and res["mean_tpot_ms"] > 0 and res["output_tokens_per_s"] > 0


def test_host_step_cost_counts_every_request():
    res = _load("host_step_cost").main(["--requests", "24", "--prompt-len", "100", "--steps", "10"])
    assert res["running_requests"] == 24 and res["steps"] == 10
    parts = res["schedule_ms"] + res["prepare_ms"] + res["launch_other_ms"] + res["update_ms"] + res["wait_ms"]
    assert 0 < parts <= res["ms_per_step"] * 1.05


def test_json_mode_eval_documents_conform():
    res = _load("json_mode_eval").main(["--in-process", "llama-tiny", "--num-questions", "1",
                                        "--max-tokens", "700", "--engine-arg", "device=cpu",
                                        "--engine-arg", "max_model_len=1024"])
    assert res["documents"] == 5 and res["parse_rate"] == 1.0 and res["conformance_rate"] == 1.0


def test_prefill_comparison_script_single_process():
    res = _load("prefill_sp_vs_tp").main(["--mode", "sp", "--model", "llama-tiny", "--num-prompts", "2",
                                          "--input-len", "24", "--iters", "2", "--warmup", "1",
                                          "--device", "cpu"])
    assert res["mode"] == "single" and res["prefill_tokens_per_s"] > 0


def test_serving_suite_starts_a_server_and_runs_tasks(tmp_path):
    import random
    port = random.randrange(20000, 28000)
    res = _load("serving_suite").main([
        "--model", "llama-tiny", "--quantization", "none", "--device", "cpu", "--configs", "baseline",
        "--tasks", "batch,single", "--num-prompts", "4", "--single-prompts", "2", "--input-len", "30",
        "--output-len", "6", "--vocab-size", "1000", "--port", str(port), "--ready-timeout", "120",
        "--log-dir", str(tmp_path)])
    row = res["baseline"]
    assert "error" not in row, row
    assert row["batch"]["completed"] == 4 and row["batch"]["total_token_throughput"] > 0
    assert row["single"]["mean_ttft_ms"] > 0 and row["single"]["failed"] == 0
