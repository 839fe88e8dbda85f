#!/usr/bin/env bash
# Stop the server started by start_server.sh: its exact process group, never a name pattern.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source ci/scripts/common/env.sh
source ci/scripts/common/log.sh
if [ -f "$B200_CI_PID_FILE" ]; then
  PID="$(cat "$B200_CI_PID_FILE")"
  kill "$PID" 2> /dev/null || true
  for _ in $(seq 1 30); do kill -0 "$PID" 2> /dev/null || break; sleep 1; done
  kill -9 "$PID" 2> /dev/null || true
  rm -f "$B200_CI_PID_FILE"
  log "server $PID stopped"
fi
