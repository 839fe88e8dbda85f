#!/usr/bin/env bash
# Unit tests: the CPU suite everywhere; the GPU suite when a GPU is visible (multi-GPU tests skip themselves).
set -euo pipefail
cd "$(dirname "$0")/../../.."
source ci/scripts/common/log.sh
log "CPU suite"
python -m pytest tests/ -x -q -m "not gpu"
if python -c "import torch, sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  log "GPU suite"
  python -m pytest tests/ -x -q -m gpu
else
  log "no GPU visible: GPU suite skipped"
fi
