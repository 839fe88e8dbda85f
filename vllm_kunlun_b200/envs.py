"""Typed environment registry, read lazily (no import-time side effects).

Mirrors the reference's lazy ``__getattr__`` registry (``vllm_kunlun/platforms/envs.py:34-92``) with this
framework's names.  ``envs.NAME`` evaluates the variable at access time."""
from __future__ import annotations

import os
from typing import Any, Callable

_ENV: dict[str, Callable[[], Any]] = {
    # per-rank stdout/stderr redirection to $B200_MULTI_LOGPATH/pp={p}_rank={r}.log (utils.logging)
    "B200_MULTI_LOGPATH": lambda: os.environ.get("B200_MULTI_LOGPATH", "./logs"),
    "B200_ENABLE_MULTI_LOG": lambda: os.environ.get("B200_ENABLE_MULTI_LOG", "0") == "1",
    # forward pre/post hook tracer on every nn.Module (utils.hooks)
    "B200_ENABLE_MODULE_HOOK": lambda: os.environ.get("B200_ENABLE_MODULE_HOOK", "0") == "1",
    # print every ops.* call with shapes (utils.hooks.LoggingOps)
    "B200_ENABLE_OPS_HOOK": lambda: os.environ.get("B200_ENABLE_OPS_HOOK", "0") == "1",
    # check on every decode-graph replay that the graph's input tensors still sit at the captured addresses
    "B200_GRAPH_WATCH": lambda: os.environ.get("B200_GRAPH_WATCH", "0") == "1",
    # NVTX ranges around layers / ops
    "B200_NVTX": lambda: os.environ.get("B200_NVTX", "0") == "1",
    # programmatic dependent launch on decode-path kernels (read by the C++ side too)
    "B200_PDL": lambda: os.environ.get("B200_PDL", "1") != "0",
    # 16 KB weight tiles per CTA that a decode-shaped GEMM pulls into L2 ahead of its smem ring (read by the C++ side; measured slower than off)
    "B200_GEMM_L2_PREFETCH": lambda: int(os.environ.get("B200_GEMM_L2_PREFETCH", "0")),
    # decode-sized GEMMs on the cluster split-K kernel / its peer-push epilogue under TP / tcgen05 decode attention
    "B200_DECODE_GEMM": lambda: os.environ.get("B200_DECODE_GEMM", "1") != "0",
    "B200_GEMM_PUSH": lambda: os.environ.get("B200_GEMM_PUSH", "1") != "0",
    "B200_ATTN_UMMA": lambda: os.environ.get("B200_ATTN_UMMA", "1") != "0",
    # host-side rank handshake every N engine steps (0 = off) and how long to wait for a silent peer
    "B200_HEALTH_CHECK_INTERVAL": lambda: int(os.environ.get("B200_HEALTH_CHECK_INTERVAL", "0")),
    "B200_HEALTH_TIMEOUT_S": lambda: float(os.environ.get("B200_HEALTH_TIMEOUT_S", "30")),
    # gated activation inside the gate/up GEMM epilogue (interleaved weight tiles); decode attention merging its own
    # split-KV partials (read by the C++ side)
    "B200_FUSE_ACT": lambda: os.environ.get("B200_FUSE_ACT", "1") != "0",
    "B200_ATTN_FUSE_MERGE": lambda: os.environ.get("B200_ATTN_FUSE_MERGE", "1") != "0",
    # low-latency all-reduce (data + flag in one 8-byte unit) for payloads up to 256 KB
    "B200_AR_LL": lambda: os.environ.get("B200_AR_LL", "1") != "0",
    # MoE decode: one-launch permute (+ fp8 quantisation) and fused activation + quantiser for small batches
    "B200_MOE_SMALL_FUSION": lambda: os.environ.get("B200_MOE_SMALL_FUSION", "1") != "0",
    # peer-memory collectives (one-shot all-reduce, fused GEMM+collectives)
    "B200_PEER_COLLECTIVES": lambda: os.environ.get("B200_PEER_COLLECTIVES", "1") != "0",
    # exponential-race sampling with a cached noise tensor (the reference's FAST_RANDOM_SAMPLE)
    "B200_FAST_RANDOM_SAMPLE": lambda: os.environ.get("B200_FAST_RANDOM_SAMPLE", "0") == "1",
    # expert parallelism: route each rank's slice of the tokens through the dispatch / combine kernels instead of
    # computing local experts over replicated tokens; capacity = tokens per step the exchange buffers are sized for
    "B200_EP_A2A": lambda: os.environ.get("B200_EP_A2A", "0") == "1",
    "B200_EP_A2A_MAX_TOKENS": lambda: int(os.environ.get("B200_EP_A2A_MAX_TOKENS", "8192")),
    # MLA prefill in the up-projected 192 / 128 form for requests with many new tokens (0: absorbed form everywhere)
    "B200_MLA_PREFILL_FORM": lambda: os.environ.get("B200_MLA_PREFILL_FORM", "1") != "0",
    # gated delta rule of requests with >= 64 new tokens in the chunked form (batched products per 64-token chunk)
    "B200_GDN_CHUNKED": lambda: os.environ.get("B200_GDN_CHUNKED", "0") == "1",
    # the chat endpoint fetches http(s) image URLs (off: only data: URIs and local files are read)
    "B200_ALLOW_REMOTE_IMAGES": lambda: os.environ.get("B200_ALLOW_REMOTE_IMAGES", "0") == "1",
    # bounded-wait budget of cross-GPU spins (iterations)
    "B200_SPIN_LIMIT": lambda: int(os.environ.get("B200_SPIN_LIMIT", str(1 << 22))),
}


def __getattr__(name: str):
    if name in _ENV:
        return _ENV[name]()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return list(_ENV)


def describe() -> dict:
    return {k: v() for k, v in _ENV.items()}
