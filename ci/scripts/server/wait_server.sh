#!/usr/bin/env bash
# Wait until the server started by start_server.sh answers /health; fail early when its process is gone.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source ci/scripts/common/env.sh
source ci/scripts/common/log.sh
[ -f "$B200_CI_PID_FILE" ] || die "no pid file: start the server first"
PID="$(cat "$B200_CI_PID_FILE")"
for i in $(seq 1 "$B200_CI_READY_TIMEOUT_S"); do
  if curl -sf "http://127.0.0.1:${B200_CI_PORT}/health" > /dev/null; then log "server ready after ${i}s"; exit 0; fi
  if ! kill -0 "$PID" 2> /dev/null; then tail -n 60 "$B200_CI_SERVER_LOG" >&2; die "server process $PID exited"; fi
  sleep 1
done
tail -n 60 "$B200_CI_SERVER_LOG" >&2
die "server not ready after ${B200_CI_READY_TIMEOUT_S}s"
