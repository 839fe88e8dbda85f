#!/usr/bin/env bash
# Serving perf check: the headline shape (16 concurrent requests, 2048 in / 2048 out) against a running server.
set -euo pipefail
PORT="${1:-8000}"
python benchmarks/bench_serving.py --port "$PORT" --num-prompts "${NUM_PROMPTS:-16}" --max-concurrency "${CONCURRENCY:-16}" \
  --random-input-len "${INPUT_LEN:-2048}" --random-output-len "${OUTPUT_LEN:-2048}" | tee perf.json
