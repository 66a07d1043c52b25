#!/usr/bin/env bash
# Replay a request trace against the server started by server.sh and write one CSV row per
# request (TTFT, TPOT, end-to-end latency), then print the percentiles.
#
#   examples/reproducibility/client.sh TRACE.jsonl [MODEL] [OUT.csv]
#   BASE_URL=http://127.0.0.1:8000,http://127.0.0.1:8001 examples/reproducibility/client.sh ...
#
# A public trace in CSV form is converted first with
#   python benchmarks/trace_tools.py convert IN.csv TRACE.jsonl --to-min 15
set -euo pipefail
here=$(cd "$(dirname "$0")/../.." && pwd)
trace=${1:?trace file}
model=${2:-llama-3.3-70b}
out=${3:-replay_output.csv}
python "$here/benchmarks/trace_replay.py" --base-url "${BASE_URL:-http://127.0.0.1:8000}" --model "$model" \
  --trace-dataset-path "$trace" --csv "$out"
python "$here/benchmarks/trace_tools.py" summarize "$out"
