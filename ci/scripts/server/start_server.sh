#!/usr/bin/env bash
# Start the OpenAI-compatible server in the background (one process per GPU under torch.distributed.run when the
# job uses more than one GPU).  usage: start_server.sh [extra server args...]
set -euo pipefail
cd "$(dirname "$0")/../../.."
source ci/scripts/common/env.sh
source ci/scripts/common/log.sh
ARGS=(--model "$B200_CI_MODEL" --port "$B200_CI_PORT" --max-model-len "$B200_CI_MAX_MODEL_LEN"
      --tensor-parallel-size "$B200_CI_TP" "$@")
if [ "$B200_CI_TP" -gt 1 ]; then
  LAUNCH=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$B200_CI_TP" --master-addr 127.0.0.1
          --master-port "${B200_CI_MASTER_PORT:-29555}" -m vllm_kunlun_b200.entrypoints.openai_server)
else
  LAUNCH=(python -m vllm_kunlun_b200.entrypoints.openai_server)
fi
log "starting: ${LAUNCH[*]} ${ARGS[*]}"
"${LAUNCH[@]}" "${ARGS[@]}" > "$B200_CI_SERVER_LOG" 2>&1 &
echo $! > "$B200_CI_PID_FILE"
log "server pid $(cat "$B200_CI_PID_FILE"), log $B200_CI_SERVER_LOG"
