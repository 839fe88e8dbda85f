#!/usr/bin/env bash
# Settings shared by the CI scripts; every value can be overridden from the environment of the job.
export B200_CI_MODEL="${B200_CI_MODEL:-llama-3.1-8b}"          # preset name or checkpoint directory
export B200_CI_PORT="${B200_CI_PORT:-8000}"
export B200_CI_TP="${B200_CI_TP:-1}"                           # tensor-parallel size (= GPUs of the job)
export B200_CI_MAX_MODEL_LEN="${B200_CI_MAX_MODEL_LEN:-8192}"
export B200_CI_SERVER_LOG="${B200_CI_SERVER_LOG:-server.log}"
export B200_CI_PID_FILE="${B200_CI_PID_FILE:-server.pid}"
export B200_CI_READY_TIMEOUT_S="${B200_CI_READY_TIMEOUT_S:-900}"
export B200_CI_RESULTS="${B200_CI_RESULTS:-ci_results}"
export MASTER_ADDR="${MASTER_ADDR:-127.0.0.1}"                  # single-node rendezvous; hostnames may not resolve
mkdir -p "$B200_CI_RESULTS"
