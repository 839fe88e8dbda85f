"""Logger set-up and per-rank output redirection.

The reference redirects each rank's stdout/stderr to ``$VLLM_MULTI_LOGPATH/pp={0|1}_rank={tp}.log`` by
wrapping ``ensure_model_parallel_initialized`` (``vllm_kunlun/utils.py:26-77``); here it is an explicit
call made after the parallel state exists."""
from __future__ import annotations

import logging
import os
import sys

_FMT = "%(levelname)s %(asctime)s [%(name)s:%(lineno)d] %(message)s"


def init_logger(name: str = "vllm_kunlun_b200", level: int = logging.INFO) -> logging.Logger:
    log = logging.getLogger(name)
    if not log.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(_FMT, datefmt="%m-%d %H:%M:%S"))
        log.addHandler(h)
        log.setLevel(level)
        log.propagate = False
    return log


def redirect_rank_output(log_dir: str | None = None, pp_rank: int = 0, tp_rank: int = 0):
    """Send this process's stdout / stderr to ``<log_dir>/pp={pp}_rank={tp}.log``; returns the path."""
    from .. import envs
    log_dir = log_dir or envs.B200_MULTI_LOGPATH
    os.makedirs(log_dir, exist_ok=True)
    path = os.path.join(log_dir, f"pp={pp_rank}_rank={tp_rank}.log")
    f = open(path, "a", buffering=1)
    os.dup2(f.fileno(), sys.stdout.fileno())
    os.dup2(f.fileno(), sys.stderr.fileno())
    return path
