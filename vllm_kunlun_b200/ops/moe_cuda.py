"""CUDA MoE path: routing -> permute -> grouped GEMM -> act -> grouped GEMM -> weighted un-permute.

Kernels: ``csrc/moe/moe.cu`` (route / count / scan / scatter / un-permute / fp8 quant) and
``csrc/gemm/gemm_grouped.cu`` (tcgen05 grouped GEMM, bf16 or fp8 block-scaled).  All shapes are
static in the token count (``T * k`` permuted rows, invalid rows masked by ``lod``), so the whole
block can sit inside a captured CUDA graph."""
from __future__ import annotations

import torch

from . import _ext

_MODES = {"softmax": 0, "sigmoid": 1, "softmax_after_topk": 2}
_STATE: dict = {}


def moe_route_cuda(logits, k, scoring, renormalize, bias, n_group, topk_group, scale):
    w, ids = _ext.C().moe_route(logits, bias, k, _MODES[scoring], renormalize, n_group, topk_group, scale)
    return w, ids


SMALL_BATCH_FUSION = [__import__("os").environ.get("B200_MOE_SMALL_FUSION", "1") != "0"]
_SMALL = []


def _small_pairs() -> int:
    if not _SMALL:
        _SMALL.append(int(_ext.C().moe_small_pairs()))
    return _SMALL[0]


def _state(device, e_local: int):
    key = (str(device), e_local)
    if key not in _STATE:
        _STATE[key] = torch.zeros(2 * e_local, dtype=torch.int32, device=device)
    return _STATE[key]


def fused_moe_cuda(x, w13, w2, topk_weights, topk_ids, act="silu", b13=None, b2=None, w13_scale=None, w2_scale=None,
                   block=(128, 128), expert_map=None):
    from . import act_and_mul
    C = _ext.C()
    T, H = x.shape
    k = topk_ids.shape[1]
    E_local = w13.shape[0]
    E_global = expert_map.shape[0] if expert_map is not None else E_local
    fp8 = w13_scale is not None
    small = 0 < T * k <= _small_pairs() and SMALL_BATCH_FUSION[0]
    if small:
        # decode-sized batch: count + scan + scatter (+ fp8 quantisation of the rows) in one launch
        xs, pos, lod, st = C.moe_prepare_small(x, topk_ids.contiguous(), expert_map, E_local, E_global, fp8)
        q = xs
    else:
        xs, pos, lod = C.moe_permute(x, topk_ids.contiguous(), expert_map, E_local, E_global, _state(x.device, E_local))
        if fp8:
            q, st = C.quant_fp8_group(xs, False, lod[E_local:], 4)
    M = xs.shape[0]
    h = torch.empty(M, w13.shape[1], dtype=x.dtype, device=x.device)
    if fp8:
        C.grouped_gemm(h, q, w13.view(torch.uint8), lod, b13, st, w13_scale, 0)
    else:
        C.grouped_gemm(h, xs, w13, lod, b13, None, None, 0)
    y = torch.empty(M, H, dtype=x.dtype, device=x.device)
    if fp8:
        if act in ("silu", "gelu_tanh") and SMALL_BATCH_FUSION[0]:
            q2, st2 = C.act_mul_quant_fp8(h, 0 if act == "silu" else 1, lod[E_local:])  # activation + quantiser fused
        else:
            q2, st2 = C.quant_fp8_group(act_and_mul(h, act), False, lod[E_local:], 4)
        C.grouped_gemm(y, q2, w2.view(torch.uint8), lod, b2, st2, w2_scale, 0)
    else:
        C.grouped_gemm(y, act_and_mul(h, act), w2, lod, b2, None, None, 0)
    out = torch.empty(T, H, dtype=x.dtype, device=x.device)
    C.moe_unpermute(out, y, pos, topk_weights.contiguous())
    return out
