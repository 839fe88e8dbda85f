"""NVTX ranges and profiler windows (the reference documents ``xtorch_ops.kunlun_profiler_start()/end()``
and layer-wise NVTX around compiled modules, ``compilation/wrapper.py:92-106``)."""
from __future__ import annotations

import contextlib

import torch


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool | None = None):
    if enabled is None:
        from .. import envs
        enabled = envs.B200_NVTX
    on = bool(enabled) and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def profiler_window():
    """cudaProfilerStart/Stop around a region (use with ``ncu --profile-from-start off``)."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    try:
        yield
    finally:
        if on:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()


def weak_ref_tensor(t: torch.Tensor) -> torch.Tensor:
    """Alias of a CUDA tensor that does not own its storage (``csrc/utils.cpp:4-32`` of the reference):
    lets a CUDA-graph runner keep output handles without pinning allocations."""
    if not t.is_cuda:
        return t
    from ..ops import _ext
    return _ext.C().weak_ref_tensor(t)
