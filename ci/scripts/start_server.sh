#!/usr/bin/env bash
# Start the OpenAI-compatible server in the background and wait until it answers /health.
# usage: ci/scripts/start_server.sh <model-or-preset> [port] [extra server args...]
set -euo pipefail
MODEL="${1:?model path or preset name}"; PORT="${2:-8000}"; shift $(( $# > 1 ? 2 : 1 ))
LOG="${SERVER_LOG:-server.log}"
python -m vllm_kunlun_b200.entrypoints.openai_server --model "$MODEL" --port "$PORT" "$@" > "$LOG" 2>&1 &
echo $! > server.pid
for i in $(seq 1 "${READY_TIMEOUT_S:-600}"); do
  if curl -sf "http://127.0.0.1:${PORT}/health" > /dev/null; then echo "server ready after ${i}s"; exit 0; fi
  if ! kill -0 "$(cat server.pid)" 2> /dev/null; then echo "server exited"; tail -50 "$LOG"; exit 1; fi
  sleep 1
done
echo "server not ready in time"; tail -50 "$LOG"; exit 1
