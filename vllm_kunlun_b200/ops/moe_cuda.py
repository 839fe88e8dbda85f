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
    xs, pos, lod = C.moe_permute(x, topk_ids.contiguous(), expert_map, E_local, E_global, _state(x.device, E_local))
    M = xs.shape[0]
    fp8 = w13_scale is not None
    h = torch.empty(M, w13.shape[1], dtype=x.dtype, device=x.device)
    if fp8:
        q, st = C.quant_fp8_group(xs, False, lod[E_local:], 4)
        C.grouped_gemm(h, q, w13.view(torch.uint8), lod, b13, st, w13_scale, 0)
    else:
        C.grouped_gemm(h, xs, w13, lod, b13, None, None, 0)
    a = act_and_mul(h, act)
    y = torch.empty(M, H, dtype=x.dtype, device=x.device)
    if fp8:
        q2, st2 = C.quant_fp8_group(a, False, lod[E_local:], 4)
        C.grouped_gemm(y, q2, w2.view(torch.uint8), lod, b2, st2, w2_scale, 0)
    else:
        C.grouped_gemm(y, a, w2, lod, b2, None, None, 0)
    out = torch.empty(T, H, dtype=x.dtype, device=x.device)
    C.moe_unpermute(out, y, pos, topk_weights.contiguous())
    return out
