#!/usr/bin/env bash
# log "message": time-stamped line on stderr, so that stdout stays machine-readable (JSON results)
log() { printf '[%s] %s\n' "$(date -u +%H:%M:%S)" "$*" >&2; }
die() { log "ERROR: $*"; exit 1; }
