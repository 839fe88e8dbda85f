"""fp32 PyTorch oracles: MoE routing, permutation, grouped GEMM, whole fused MoE.

Stage graph of the reference (``ops/_kunlun_ops.py:397-637``): route -> sort/permute ->
``moe_fc(w13)`` -> ``silu_and_mul`` -> ``moe_fc(w2)`` -> ``moe_post``.
"""
from __future__ import annotations

import torch

from .basic import dequant_fp8_block, gelu_tanh_and_mul, quant_fp8_per_group, silu_and_mul, swigluoai_and_mul


def route_softmax_topk(logits, k: int, renormalize: bool = True):
    """``_C::moe_softmax_topk_norm`` / ``_C::moe_softmax_topk`` (``ops/_custom_ops.py:781-802,1084-1107``)."""
    p = torch.softmax(logits.float(), -1)
    w, ids = torch.topk(p, k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, ids.to(torch.int32)


def route_topk_then_softmax(logits, k: int):
    """GPT-OSS routing: top-k on raw logits, softmax over the selected k."""
    v, ids = torch.topk(logits.float(), k, dim=-1)
    return torch.softmax(v, -1), ids.to(torch.int32)


def route_sigmoid_group_topk(logits, bias, k: int, n_group: int, topk_group: int,
                             renormalize: bool = True, scale: float = 1.0):
    """``_C::moe_sigmoid_group_topk_norm`` (``ops/_custom_ops.py:1351-1394``): DeepSeek-V3 routing.
    Scores = sigmoid(logits); selection uses ``scores + bias``; each group is ranked by the sum of
    its top-2 biased scores, the best ``topk_group`` groups stay; final weights are the *unbiased*
    scores of the chosen experts, normalised and multiplied by ``scale``."""
    T, E = logits.shape
    s = torch.sigmoid(logits.float())
    sel = s + bias.float() if bias is not None else s
    g = sel.reshape(T, n_group, E // n_group)
    gscore = g.topk(min(2, E // n_group), -1).values.sum(-1)
    gidx = gscore.topk(topk_group, -1).indices
    gmask = torch.zeros(T, n_group, dtype=torch.bool).scatter_(1, gidx, True)
    masked = g.masked_fill(~gmask.unsqueeze(-1), float("-inf")).reshape(T, E)
    ids = masked.topk(k, -1).indices
    w = s.gather(1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scale, ids.to(torch.int32)


def moe_permute(x, topk_ids, num_experts: int):
    """``gen_block_statistic`` + ``moe_pre_sorted`` (``ops/_custom_ops.py:1123-1185``): expand each
    token ``k`` times and sort by expert.  Returns ``(x_sorted [T*k, H], sorted_idx [T*k]``
    (flat ``token*k + slot`` ids in sorted order), ``lod [E+1])``."""
    flat = topk_ids.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    lod = torch.zeros(num_experts + 1, dtype=torch.int32)
    lod[1:] = counts.cumsum(0)
    k = topk_ids.shape[1]
    return x[order // k], order.to(torch.int32), lod


def grouped_gemm(x_sorted, w, lod, bias=None):
    """``_C::moe_fc`` (``ops/_custom_ops.py:1204-1287``): ``y[r] = x[r] @ w[e].T`` for rows of expert ``e``.
    ``w [E, N, K]``."""
    out = torch.zeros(x_sorted.shape[0], w.shape[1], dtype=torch.float32)
    for e in range(w.shape[0]):
        s, t = int(lod[e]), int(lod[e + 1])
        if t > s:
            out[s:t] = x_sorted[s:t].float() @ w[e].float().T
            if bias is not None:
                out[s:t] += bias[e].float()
    return out.to(x_sorted.dtype)


def moe_unpermute(y_sorted, sorted_idx, topk_weights, num_tokens: int):
    """``_C::moe_post`` (``ops/_custom_ops.py:1316-1335``): un-permute + weighted sum over top-k."""
    k = topk_weights.shape[1]
    buf = torch.zeros(num_tokens * k, y_sorted.shape[1], dtype=torch.float32)
    buf[sorted_idx.long()] = y_sorted.float()
    return (buf.reshape(num_tokens, k, -1) * topk_weights.float().unsqueeze(-1)).sum(1).to(y_sorted.dtype)


def fused_moe(x, w13, w2, topk_weights, topk_ids, act: str = "silu", b13=None, b2=None,
              w13_scale=None, w2_scale=None, block=(128, 128), expert_map=None):
    """Whole MoE block on routed tokens.  With ``w13_scale``/``w2_scale`` the weights are fp8
    block-128 and activations are re-quantised per 1x128 group before each GEMM (the W8A8 pipeline
    of ``quantization/compressed_tensors/compressed_tensors_moe.py:122-291`` restated for fp8).
    ``expert_map [E_global] -> local id or -1`` restricts to this rank's experts (EP)."""
    T, k = topk_ids.shape
    E = w13.shape[0]
    ids = topk_ids.long()
    wts = topk_weights.float()
    if expert_map is not None:
        local = expert_map.long()[ids]
        wts = torch.where(local >= 0, wts, torch.zeros_like(wts))
        ids = local.clamp(min=0)
    if w13_scale is not None:
        w13f = dequant_fp8_block(w13, w13_scale, block)
        w2f = dequant_fp8_block(w2, w2_scale, block)
    else:
        w13f, w2f = w13.float(), w2.float()
    xs, order, lod = moe_permute(x, ids.to(torch.int32), E)

    def _q(t):
        if w13_scale is None:
            return t
        q, s = quant_fp8_per_group(t, block[1])
        return (q.float().reshape(*s.shape, block[1]) * s.unsqueeze(-1)).reshape(t.shape).to(t.dtype)

    h = grouped_gemm(_q(xs), w13f, lod, b13)
    h = {"swigluoai": swigluoai_and_mul, "gelu_tanh": gelu_tanh_and_mul}.get(act, silu_and_mul)(h)
    y = grouped_gemm(_q(h), w2f, lod, b2)
    return moe_unpermute(y, order, wts, T)
