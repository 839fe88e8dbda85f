#!/usr/bin/env bash
# Stop the server started by start_server.sh (exact PID, never by pattern).
set -euo pipefail
[ -f server.pid ] && kill "$(cat server.pid)" 2> /dev/null || true
rm -f server.pid
