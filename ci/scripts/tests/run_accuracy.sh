#!/usr/bin/env bash
# Accuracy smoke against the running server: deterministic greedy completions, logprob sanity, chat template path.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source ci/scripts/common/env.sh
source ci/scripts/common/log.sh
log "accuracy checks against port $B200_CI_PORT"
python ci/scripts/run_accuracy.py --port "$B200_CI_PORT" | tee "$B200_CI_RESULTS/accuracy.json"
