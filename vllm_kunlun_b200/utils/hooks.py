"""Tracing hooks: module forward tracer, op-call logger, stage timer.

Counterparts of the reference's opt-in debug module (``vllm_kunlun/utils.py``): stage markers
"First Token / Per Token Start/End" (``:80-123``), ``register_module_forward_(pre_)hook`` indentation
tracer (``:126-196``), ``LoggingDispatchMode`` printing every op (``:199-232``)."""
from __future__ import annotations

import contextlib
import functools
import time
from typing import Callable, Optional

import torch


class ModuleTracer:
    """Prints an indented call tree of ``nn.Module.forward`` with output shapes."""

    def __init__(self, root: torch.nn.Module, sink: Callable[[str], None] = print, max_depth: int = 6):
        self.root, self.sink, self.max_depth = root, sink, max_depth
        self.depth = 0
        self._handles = []

    def __enter__(self):
        for name, m in self.root.named_modules():
            self._handles.append(m.register_forward_pre_hook(functools.partial(self._pre, name)))
            self._handles.append(m.register_forward_hook(functools.partial(self._post, name)))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles.clear()

    def _pre(self, name, mod, args):
        if self.depth < self.max_depth:
            self.sink("  " * self.depth + f"-> {name or '<root>'} ({type(mod).__name__})")
        self.depth += 1

    def _post(self, name, mod, args, out):
        self.depth -= 1
        if self.depth < self.max_depth:
            shp = tuple(out.shape) if isinstance(out, torch.Tensor) else type(out).__name__
            self.sink("  " * self.depth + f"<- {name or '<root>'} {shp}")


class LoggingOps:
    """Wraps every public function of :mod:`vllm_kunlun_b200.ops` to log its tensor arguments."""

    def __init__(self, sink: Callable[[str], None] = print):
        self.sink = sink
        self._saved = {}

    def __enter__(self):
        from .. import ops
        for name in dir(ops):
            fn = getattr(ops, name)
            if name.startswith("_") or not callable(fn) or isinstance(fn, type) or getattr(fn, "__module__", "") != ops.__name__:
                continue
            self._saved[name] = fn
            setattr(ops, name, self._wrap(name, fn))
        return self

    def __exit__(self, *exc):
        from .. import ops
        for name, fn in self._saved.items():
            setattr(ops, name, fn)
        self._saved.clear()

    def _wrap(self, name, fn):
        @functools.wraps(fn)
        def inner(*a, **k):
            shapes = [tuple(x.shape) if isinstance(x, torch.Tensor) else x for x in a
                      if isinstance(x, (torch.Tensor, int, float, bool, str))]
            self.sink(f"ops.{name}{shapes}")
            return fn(*a, **k)
        return inner


class StageTimer:
    """First-token / per-token stage markers around engine steps."""

    def __init__(self, sink: Optional[Callable[[str], None]] = print):
        self.sink = sink
        self.records = []

    @contextlib.contextmanager
    def stage(self, name: str, sync: bool = False):
        if sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        if self.sink:
            self.sink(f"[stage] {name} start")
        try:
            yield
        finally:
            if sync and torch.cuda.is_available():
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            self.records.append((name, dt))
            if self.sink:
                self.sink(f"[stage] {name} end {dt * 1e3:.3f} ms")


class GraphInputWatcher:
    """Guards the tensors a captured CUDA graph reads: their addresses (and shapes) must not change between capture
    and replay, or the graph silently reads stale memory.  Counterpart of the reference's ``CUDAGraphInnerWatcher``
    (``vllm_kunlun/utils.py:235-288``), which logs tensor addresses inside compiled graphs for the same purpose.

        watcher = GraphInputWatcher()
        watcher.capture("decode_b16", {"ids": ids, "block_tables": bt})
        ...
        watcher.check("decode_b16", {"ids": ids, "block_tables": bt})   # raises on a moved / reshaped tensor
    """

    def __init__(self):
        self._seen: dict = {}

    @staticmethod
    def _sig(t: torch.Tensor):
        return (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype)

    def capture(self, key: str, tensors: dict) -> None:
        self._seen[key] = {n: self._sig(t) for n, t in tensors.items() if isinstance(t, torch.Tensor)}

    def check(self, key: str, tensors: dict) -> None:
        ref = self._seen.get(key)
        if ref is None:
            raise KeyError(f"graph {key!r} was never captured")
        for n, t in tensors.items():
            if isinstance(t, torch.Tensor) and n in ref and self._sig(t) != ref[n]:
                raise RuntimeError(f"input {n!r} of captured graph {key!r} changed: {ref[n]} -> {self._sig(t)}")
