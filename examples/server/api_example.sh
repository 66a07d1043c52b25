#!/bin/sh
# REST walk-through against `python -m arcticinference_b200.server.cli --port 8000`.
BASE=${BASE:-http://127.0.0.1:8000}
curl -s -X POST $BASE/init -H 'content-type: application/json' \
  -d '{"config": {"model": "llama-3.1-8b", "quantization": "fp8", "max_model_len": 8192}, "model_id": "m"}'
curl -s -X POST $BASE/generate -H 'content-type: application/json' \
  -d '{"prompts": ["Hello", [1, 2, 3]], "sampling_params": {"max_tokens": 16}, "routing_key": "session-1"}'
curl -s $BASE/status
curl -s -X POST $BASE/sleep -H 'content-type: application/json' -d '{"model_id": "m", "level": 2}'
curl -s -X POST $BASE/wake_up -H 'content-type: application/json' -d '{"model_id": "m", "tags": ["weights"]}'
# ... POST /sync_weights while only the weights are resident ...
curl -s -X POST $BASE/wake_up -H 'content-type: application/json' -d '{"model_id": "m", "tags": ["kv_cache"]}'
curl -s $BASE/metrics
curl -s -X POST "$BASE/shutdown?model_id=m"
