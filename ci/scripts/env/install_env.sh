#!/usr/bin/env bash
# Prepare a job's checkout: check the toolchain and the GPUs, build the sm_100a extension in-tree, write the
# entry-point metadata that lets an installed vLLM find the plugin from the checkout, and import the package.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source ci/scripts/common/env.sh
source ci/scripts/common/log.sh
command -v nvcc > /dev/null || die "nvcc not on PATH (CUDA 12.8+ with sm_100a support is required)"
python - <<'PY' || die "python environment incomplete"
import sys, torch
assert sys.version_info >= (3, 10), sys.version
print("torch", torch.__version__, "cuda", torch.version.cuda)
PY
if command -v nvidia-smi > /dev/null; then
  log "GPUs (read-only query; no clocks, power limits or modes are touched):"
  nvidia-smi --query-gpu=index,name,memory.total,clocks.max.sm --format=csv >&2 || true
  n=$(nvidia-smi -L | wc -l)
  [ "$n" -ge "$B200_CI_TP" ] || die "job wants $B200_CI_TP GPUs, the host shows $n"
else
  log "no nvidia-smi: building only (nvcc cross-compiles without a GPU)"
fi
log "building the extension"
python -m vllm_kunlun_b200.build
python - <<'PY'
import vllm_kunlun_b200
from vllm_kunlun_b200.ops import _ext
assert _ext.so_path() is not None, "extension did not build"
print("extension:", _ext.so_path())
PY
log "environment ready"
