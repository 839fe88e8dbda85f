#!/usr/bin/env bash
# Serving performance matrix against the running server: every (concurrency, input x output length) pair of the two
# lists below, one JSON line per case in $B200_CI_RESULTS/perf.jsonl.  The headline case of the published numbers is
# 16 concurrent requests with 2048 input and 2048 output tokens.
#   CONCURRENCIES="1 4 16" DIMENSIONS="1024x1024 2048x2048" ci/scripts/tests/run_performance.sh
set -euo pipefail
cd "$(dirname "$0")/../../.."
source ci/scripts/common/env.sh
source ci/scripts/common/log.sh
read -r -a CONC <<< "${CONCURRENCIES:-16}"
read -r -a DIMS <<< "${DIMENSIONS:-2048x2048}"
OUT="$B200_CI_RESULTS/perf.jsonl"
: > "$OUT"
total=$(( ${#CONC[@]} * ${#DIMS[@]} )); k=0
for c in "${CONC[@]}"; do
  for d in "${DIMS[@]}"; do
    k=$((k + 1))
    in_len="${d%x*}"; out_len="${d#*x}"
    log "case $k/$total: concurrency $c, $in_len in / $out_len out"
    python benchmarks/bench_serving.py --port "$B200_CI_PORT" --num-prompts "$(( c * ${ROUNDS:-1} ))" \
      --max-concurrency "$c" --random-input-len "$in_len" --random-output-len "$out_len" | tail -n 1 | tee -a "$OUT"
  done
done
log "wrote $OUT"
