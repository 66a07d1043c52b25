#!/usr/bin/env bash
# Serve one model for the trace replay in one of three layouts over the GPUs of this node
# (the comparison of the reference's benchmark/reproducibility/server.sh: shift parallelism
# against tensor parallelism against replicas).
#
#   examples/reproducibility/server.sh [shift|tp|dp] [MODEL] [GPUS]
set -euo pipefail
layout=${1:-shift}
model=${2:-llama-3.3-70b}        # or qwen3-32b, a checkpoint directory, ...
gpus=${3:-8}
common="--quantization fp8 --no-enable-prefix-caching --max-num-batched-tokens 131072 --port 8000"
case "$layout" in
  shift)
    exec python -m arcticinference_b200.cli serve "$model" $common \
      --ulysses-sequence-parallel-size "$gpus" --enable-shift-parallel ;;
  tp)
    exec python -m arcticinference_b200.cli serve "$model" $common \
      --tensor-parallel-size "$gpus" ;;
  dp)
    # independent single-GPU servers on ports 8000..; the client spreads requests over them
    # (client.sh with BASE_URL=http://127.0.0.1:8000,http://127.0.0.1:8001,...)
    pids=()
    trap 'kill "${pids[@]}" 2>/dev/null || true' EXIT
    for ((i = 0; i < gpus; i++)); do
      CUDA_VISIBLE_DEVICES=$i python -m arcticinference_b200.cli serve "$model" \
        --quantization fp8 --no-enable-prefix-caching --max-num-batched-tokens 131072 \
        --port $((8000 + i)) &
      pids+=($!)
    done
    wait ;;
  *)
    echo "unknown layout: $layout" >&2; exit 2 ;;
esac
