"""CUDA GEMM entry: ``y = x @ W.T (+ b)`` on the tcgen05 kernel (``csrc/gemm/gemm_bf16.cu``).

The reference runs dense linears through ``F.linear`` on the vendor BLAS
(``fc_cdnn_infer`` in its profiles, ``docs/.../profiling.md:420``); no library GEMM is used here.
"""
from __future__ import annotations

import os

import torch

from . import _ext

LAUNCHES = 0
# Calls of at most 32 rows go to the cluster split-K kernel (csrc/gemm/gemm_decode.cu); B200_DECODE_GEMM=0 keeps
# them on the general kernel.
DECODE_GEMM = [os.environ.get("B200_DECODE_GEMM", "1") != "0"]
PEER = None  # PeerBuffers of the tensor-parallel group once its sequence-parallel buffers exist


ACT_CODES = {None: 0, "silu": 1, "gelu_tanh": 2, "swigluoai": 3}


def interleave_gate_up(w: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Row order of a ``[gate | up]`` projection for the fused activation epilogue: per 128-row weight tile,
    64 gate rows followed by the 64 up rows of the same features (``inverse`` undoes it)."""
    n2 = w.shape[0]
    n = n2 // 2
    assert n % 64 == 0
    if inverse:
        v = w.reshape(n // 64, 2, 64, *w.shape[1:])
        return torch.cat([v[:, 0].reshape(n, *w.shape[1:]), v[:, 1].reshape(n, *w.shape[1:])], 0)
    g, u = w[:n].reshape(n // 64, 1, 64, *w.shape[1:]), w[n:].reshape(n // 64, 1, 64, *w.shape[1:])
    return torch.cat([g, u], 1).reshape(n2, *w.shape[1:]).contiguous()


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, bias=None, out=None, splits: int = 0, bn: int = 0,
              stages: int = 0, ctas_per_sm: int = 0, act=None):
    """``act``: gated activation fused into the epilogue; ``weight`` (and ``bias``) rows are then interleaved per
    tile (:func:`interleave_gate_up`) and the output has ``N / 2`` features."""
    global LAUNCHES
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    N = weight.shape[0] // 2 if act else weight.shape[0]
    if out is None:
        out = torch.empty(x2.shape[0], N, dtype=x.dtype, device=x.device)
    out2 = out.reshape(-1, N)
    if PEER is not None and PEER.sp_pending is not None:
        ag_bn = PEER.sp_consume(x2)
        if ag_bn:  # gathered activations: the producer waits per token tile, tiles must match the counters
            bn, splits = ag_bn, 1
            _ext.C().gemm(out2, x2, weight, bias, splits, bn, stages, ctas_per_sm, ACT_CODES[act])
            LAUNCHES += 1
            return out.reshape(*lead, N)
    if DECODE_GEMM[0] and x2.shape[0] <= 32 and bn == 0:
        _ext.C().gemm_decode(out2, x2, weight, bias, splits, stages, ctas_per_sm, ACT_CODES[act])
    else:
        _ext.C().gemm(out2, x2, weight, bias, splits, bn, stages, ctas_per_sm, ACT_CODES[act])
    LAUNCHES += 1
    return out.reshape(*lead, N)


def gemm_decode_push(x: torch.Tensor, weight: torch.Tensor, peer, bias=None, out=None):
    """Row-parallel decode GEMM whose epilogue also pushes the partial result into every peer's low-latency
    all-reduce slot; finish with ``peer.collect_add_rmsnorm`` / ``peer.collect`` on the returned tensor."""
    global LAUNCHES
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    N = weight.shape[0]
    if out is None:
        out = torch.empty(x2.shape[0], N, dtype=x.dtype, device=x.device)
    C = _ext.C()
    C.set_gemm_decode_comm(peer.ll_ptrs, peer.ll_epochs, peer.ll_slot_bytes, peer.rank)
    C.gemm_decode(out, x2, weight, bias, 0, 0, 0, 0)
    LAUNCHES += 1
    return out


# qkv projection + split + q / k norm + rotary + cache write in one launch for decode-sized batches
# (B200_QKV_EPILOGUE=0 keeps the projection and the split / rope / cache kernel apart)
QKV_EPILOGUE = [os.environ.get("B200_QKV_EPILOGUE", "1") != "0"]


def gemm_decode_qkv(x, weight, bias, positions, cos_sin, q_w, k_w, eps, num_heads, num_kv_heads, neox, gemma,
                    kv_cache, slot_mapping):
    """``q [T, Hq * 128]`` of a batch of at most 32 tokens; K and V go straight into the paged cache."""
    global LAUNCHES
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    q = torch.empty(x2.shape[0], num_heads * 128, dtype=x.dtype, device=x.device)
    _ext.C().gemm_decode_qkv(q, x2, weight, bias, positions, cos_sin, q_w, k_w, float(eps), num_heads, num_kv_heads,
                             bool(neox), bool(gemma), kv_cache, slot_mapping)
    LAUNCHES += 1
    return q


def qkv_epilogue_ok(x, weight, head_dim, rotary_dim, kv_cache) -> bool:
    return (QKV_EPILOGUE[0] and DECODE_GEMM[0] and x.is_cuda and x.dim() == 2 and x.shape[0] <= 32 and head_dim == 128
            and rotary_dim == 128 and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype
            and weight.dim() == 2 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and x.shape[1] % 8 == 0
            and (kv_cache is None or (kv_cache.dim() == 5 and kv_cache.is_contiguous() and kv_cache.dtype == x.dtype)))


def check_status() -> None:
    """Raise if any GEMM CTA gave up on a bounded wait (a device-side status word, read on demand)."""
    code = _ext.C().gemm_status()
    if code:
        raise RuntimeError(f"tcgen05 GEMM reported a timed-out wait, code {code}")
