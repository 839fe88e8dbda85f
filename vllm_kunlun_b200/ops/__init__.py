"""Functional op layer.

Every function takes tensors and dispatches on their device: CUDA tensors go to the hand-written
sm_100a kernels in the in-tree extension (and fail loudly if it is missing); CPU tensors go to the
fp32 oracles in :mod:`vllm_kunlun_b200.ops.reference`.  This replaces the reference's two binding
layers (``vllm_kunlun/ops/_custom_ops.py`` - 54 ``torch.library.custom_op`` shims - and
``vllm_kunlun/ops/_kunlun_ops.py`` - the ``KunlunOps`` facade), which forward to closed libraries.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _ext
from .reference import attention as _ra
from .reference import basic as _rb
from .reference import misc as _rx
from .reference import moe as _rm

reference_basic = _rb
reference_attention = _ra
reference_moe = _rm
reference_misc = _rx


def _c():
    return _ext.C()


# ----------------------------------------------------------------------------- norms / activations

def rmsnorm(x, weight, eps: float, gemma: bool = False):
    if x.is_cuda:
        out = torch.empty_like(x)
        _c().rmsnorm(out, x, weight, eps, gemma)
        return out
    return _rb.rmsnorm(x, weight, eps, gemma)


def add_rmsnorm(x, residual, weight, eps: float, gemma: bool = False):
    """Returns ``(normed, new_residual)``.  On CUDA both are written in place
    (``x`` becomes the normed output, ``residual`` the sum)."""
    if x.is_cuda:
        _c().add_rmsnorm(x, residual, weight, eps, gemma)
        return x, residual
    return _rb.add_rmsnorm(x, residual, weight, eps, gemma)


def rms_norm_gated(x, z, weight, eps, norm_before_gate=True, group_size=None):
    if x.is_cuda:
        gs = group_size or x.shape[-1]
        xs, zs = x.reshape(-1, gs).contiguous(), z.reshape(-1, gs).contiguous()
        if gs != x.shape[-1]:
            return _rb.rms_norm_gated(x, z, weight, eps, norm_before_gate, group_size)
        out = torch.empty_like(xs)
        _c().rownorm(out, xs, zs, weight, eps, 2 if norm_before_gate else 3)
        return out.reshape(x.shape)
    return _rb.rms_norm_gated(x, z, weight, eps, norm_before_gate, group_size)


def l2norm(x, eps: float = 1e-6):
    if x.is_cuda:
        xc = x.contiguous()
        out = torch.empty_like(xc)
        _c().rownorm(out, xc, None, None, eps, 1)
        return out
    return _rb.l2norm(x, eps)


_ACT_CODES = {"silu": 0, "gelu_tanh": 1, "swigluoai": 2}


def act_and_mul(x, act: str = "silu"):
    if x.is_cuda:
        d = x.shape[-1] // 2
        out = torch.empty(*x.shape[:-1], d, dtype=x.dtype, device=x.device)
        _c().act_and_mul(out, x, _ACT_CODES[act])
        return out
    if act == "silu":
        return _rb.silu_and_mul(x)
    if act == "swigluoai":
        return _rb.swigluoai_and_mul(x)
    return _rb.gelu_tanh_and_mul(x)


def silu_and_mul(x):
    return act_and_mul(x, "silu")


def quick_gelu(x):
    if x.is_cuda:
        out = torch.empty_like(x)
        _c().quick_gelu(out, x)
        return out
    return _rb.quick_gelu(x)


# ----------------------------------------------------------------------------- rotary / cache

def rope(q, k, positions, cos_sin_cache, head_dim: int, neox: bool = True):
    """In-place style rotary on ``q [T, Hq*D]`` and ``k [T, Hkv*D]``; returns ``(q, k)``."""
    if q.is_cuda:
        _c().rope(q, k, positions, cos_sin_cache, head_dim, neox)
        return q, k
    rd = cos_sin_cache.shape[-1]
    return (_rb.apply_rope(q, positions, cos_sin_cache, head_dim, neox, rd),
            _rb.apply_rope(k, positions, cos_sin_cache, head_dim, neox, rd))


def mrope(q, k, positions3, cos_sin_cache, head_dim, sections, interleaved=False):
    if q.is_cuda:
        _c().mrope(q, k, positions3, cos_sin_cache, head_dim, list(sections), interleaved)
        return q, k
    return (_rb.apply_mrope(q, positions3, cos_sin_cache, head_dim, sections, interleaved),
            _rb.apply_mrope(k, positions3, cos_sin_cache, head_dim, sections, interleaved))


def reshape_and_cache(k, v, kv_cache, slot_mapping):
    if k.is_cuda:
        _c().reshape_and_cache(k, v, kv_cache, slot_mapping)
    else:
        _ra.reshape_and_cache(k, v, kv_cache, slot_mapping)


def qkv_split_norm_rope_cache(qkv, positions, cos_sin_cache, q_weight, k_weight, eps: float,
                              num_heads: int, num_kv_heads: int, head_dim: int, neox: bool,
                              kv_cache, slot_mapping, gemma: bool = False):
    """One pass over a fused qkv row: split, optional per-head q/k RMSNorm, RoPE, and the K/V
    scatter into the paged cache (``_C::split_norm_rope_neox`` + ``reshape_and_cache_flash`` of the
    reference in a single kernel).  Returns the rotated ``q [T, Hq*D]``."""
    T = qkv.shape[0]
    if qkv.is_cuda:
        q = torch.empty(T, num_heads * head_dim, dtype=qkv.dtype, device=qkv.device)
        _c().qkv_split_norm_rope_cache(q, qkv, positions, cos_sin_cache, q_weight, k_weight, eps,
                                       num_heads, num_kv_heads, head_dim, neox, gemma, kv_cache, slot_mapping)
        return q
    q, k, v = _rb.split_qknorm_rope(qkv, positions, cos_sin_cache, q_weight, k_weight, eps,
                                    num_heads, num_kv_heads, head_dim, neox, gemma)
    if kv_cache is not None:
        _ra.reshape_and_cache(k.reshape(T, num_kv_heads, head_dim), v.reshape(T, num_kv_heads, head_dim),
                              kv_cache, slot_mapping)
    return q


def concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping):
    if kv_c.is_cuda:
        _c().concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping)
    elif kv_cache.dtype == torch.uint8:
        _ra.concat_and_cache_mla_fp8(kv_c, k_pe, kv_cache, slot_mapping)
    else:
        _ra.concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping)


def indexer_k_quant_and_cache(k, k_cache, slot_mapping, ue8m0: bool = True):
    if k.is_cuda:
        _c().indexer_k_quant_and_cache(k, k_cache, slot_mapping, ue8m0)
    else:
        _ra.indexer_k_quant_and_cache(k, k_cache, slot_mapping, ue8m0)


def convert_req_index_to_global_index(req_id, block_table, token_indices, block_size: int):
    if token_indices.is_cuda:
        out = torch.empty_like(token_indices, dtype=torch.int32)
        _c().convert_req_index_to_global_index(out, req_id, block_table, token_indices, block_size)
        return out
    return _ra.convert_req_index_to_global_index(req_id, block_table, token_indices, block_size)


def copy_blocks(caches, mapping):
    if caches and caches[0].is_cuda:
        src = torch.tensor([m[0] for m in mapping], dtype=torch.int64, device=caches[0].device)
        dst = torch.tensor([m[1] for m in mapping], dtype=torch.int64, device=caches[0].device)
        for c in caches:
            _c().copy_blocks(c, src, dst)
    else:
        _ra.copy_blocks(caches, mapping)


def swap_blocks(src, dst, mapping):
    """Host<->device or device<->device block moves: one async copy per block."""
    for s, d in mapping:
        dst[d].copy_(src[s], non_blocking=True)


# ----------------------------------------------------------------------------- attention

def paged_attention(q, kv_cache, block_tables, seq_lens, query_start_loc, scale: float,
                    max_query_len: int, max_seq_len: int, window: Optional[int] = None, sinks=None,
                    seq_lens_cpu=None, query_start_loc_cpu=None, out=None, workspace=None,
                    num_decodes: int = 0, decode_query_len: int = 1, num_decode_tokens: int = 0,
                    stable_metadata: bool = False):
    """Unified varlen paged GQA attention (prefill with prefix, decode, spec-verify).

    The batch is decode-first: the first ``num_decodes`` requests have at most ``decode_query_len``
    query tokens each.  On CUDA a mixed batch is served by two launches (decode layout with
    split-KV, then the prefill layout) over views of the same tensors."""
    if q.is_cuda:
        if out is None:
            out = torch.empty(q.shape[0], q.shape[1], kv_cache.shape[-1], dtype=q.dtype, device=q.device)
        from .attention_cuda import paged_attention_cuda
        B = seq_lens.shape[0]
        if 0 < num_decodes < B:
            ndt = num_decode_tokens or num_decodes * decode_query_len
            paged_attention_cuda(out[:ndt], q[:ndt], kv_cache, block_tables[:num_decodes], seq_lens[:num_decodes],
                                 query_start_loc[:num_decodes + 1], scale, decode_query_len, max_seq_len,
                                 window, sinks, workspace, stable_metadata=stable_metadata)
            paged_attention_cuda(out, q, kv_cache, block_tables[num_decodes:], seq_lens[num_decodes:],
                                 query_start_loc[num_decodes:], scale, max_query_len, max_seq_len,
                                 window, sinks, workspace)
            return out
        return paged_attention_cuda(out, q, kv_cache, block_tables, seq_lens, query_start_loc, scale,
                                    max_query_len, max_seq_len, window, sinks, workspace,
                                    stable_metadata=stable_metadata)
    sl = seq_lens if seq_lens_cpu is None else seq_lens_cpu
    ql = query_start_loc if query_start_loc_cpu is None else query_start_loc_cpu
    return _ra.paged_attention(q, kv_cache, block_tables, sl, ql, scale, window, sinks)


def merge_attn_states(o1, lse1, o2, lse2):
    if o1.is_cuda:
        out = torch.empty_like(o1)
        lse = torch.empty_like(lse1)
        _c().merge_attn_states(out, lse, o1.contiguous(), lse1.contiguous(), o2.contiguous(), lse2.contiguous())
        return out, lse
    return _ra.merge_attn_states(o1, lse1, o2, lse2)


# ----------------------------------------------------------------------------- GEMM

def linear(x, weight, bias=None, out=None):
    """``y = x @ W.T (+ b)``, ``W [N, K]`` as stored in checkpoints.  CUDA: the tcgen05 GEMM."""
    if x.is_cuda:
        from .gemm_cuda import gemm_bf16
        return gemm_bf16(x, weight, bias, out)
    return _rb.linear(x, weight, bias)


def linear_gated_act(x, weight_interleaved, bias_interleaved=None, act: str = "silu"):
    """``act(x W_gate^T) * (x W_up^T)`` in one GEMM: the activation runs in the epilogue over weight tiles that
    hold 64 gate rows and the 64 matching up rows (CUDA only; see ``gemm_cuda.interleave_gate_up``)."""
    from .gemm_cuda import gemm_bf16, interleave_gate_up
    if x.is_cuda:
        return gemm_bf16(x, weight_interleaved, bias_interleaved, act=act)
    w = interleave_gate_up(weight_interleaved, inverse=True)
    b = None if bias_interleaved is None else interleave_gate_up(bias_interleaved, inverse=True)
    return act_and_mul(_rb.linear(x, w, b), act)


def embedding(ids, weight, vocab_start: int = 0):
    """Vocab-parallel gather: rows outside ``[vocab_start, vocab_start + rows)`` yield zeros
    (``ops/vocab_parallel_embedding.py:94-118``)."""
    if ids.is_cuda:
        out = torch.empty(ids.shape[0], weight.shape[1], dtype=weight.dtype, device=weight.device)
        _c().embedding(out, ids, weight, vocab_start)
        return out
    local = ids.long() - vocab_start
    ok = (local >= 0) & (local < weight.shape[0])
    out = weight[local.clamp(0, weight.shape[0] - 1)]
    return out * ok.unsqueeze(-1).to(out.dtype)


# ----------------------------------------------------------------------------- sampling

def argmax(logits):
    if logits.is_cuda:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
        _c().argmax(out, logits)
        return out
    return logits.float().argmax(-1)


__all__ = [n for n in dir() if not n.startswith("_")]


# ----------------------------------------------------------------------------- quantised linears

def quant_fp8_per_group(x, group: int = 128, ue8m0: bool = False):
    """Dynamic 1 x ``group`` e4m3 quantisation: ``(q, scale [..., K/group])``."""
    if x.is_cuda:
        from .quant_cuda import quant_fp8_group_cuda
        return quant_fp8_group_cuda(x, group, ue8m0)
    return _rb.quant_fp8_per_group(x, group, ue8m0)


def fp8_linear(x, w_fp8, w_scale_inv, bias=None, block=(128, 128), out_dtype=torch.bfloat16):
    """``y = x @ dequant(W).T`` with activations quantised per 1x128 group on the fly."""
    if x.is_cuda:
        from .quant_cuda import fp8_linear_cuda
        return fp8_linear_cuda(x, w_fp8, w_scale_inv, bias, block, out_dtype)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    q, s = _rb.quant_fp8_per_group(x2, block[1])
    y = _rb.fp8_block_gemm(q, s, w_fp8, w_scale_inv, block, torch.float32)
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype if out_dtype != torch.float8_e4m3fn else torch.bfloat16).reshape(*lead, -1)


W4_DECODE_ROWS = 32   # batches up to this many rows stream the packed weights through the decode GEMM


def w4_linear(x, packed, scale, zero, group: int, bias=None):
    """Linear over 4-bit weights in the packed layout of ``quantization/int4.py`` (``packed [N, K / 2]`` uint8,
    ``scale`` / ``zero [N, K / group]``): ``y = x @ ((q - zero) * scale).T (+ b)``.  CUDA: at most 32 rows run on the
    decode GEMM, which streams the packed bytes and de-quantises in the kernel; larger batches de-quantise into a
    temporary 16-bit matrix and run the 16-bit GEMM (``quantization/awq.py:124-168`` of the reference)."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x.is_cuda:
        N, K = packed.shape[0], packed.shape[1] * 2
        if x2.dtype != scale.dtype:
            x2 = x2.to(scale.dtype)
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        if 0 < x2.shape[0] <= W4_DECODE_ROWS:
            out = torch.empty(x2.shape[0], N, dtype=x2.dtype, device=x2.device)
            _c().gemm_decode_w4(out, x2, packed, scale, zero, bias, int(group), 0, 0)
            return out.reshape(*lead, N)
        w = torch.empty(N, K, dtype=scale.dtype, device=x2.device)
        _c().dequant_w4(w, packed, scale, zero, int(group))
        return linear(x2, w, bias).reshape(*lead, N)
    from ..quantization.int4 import dequant_w4
    return _rb.linear(x2, dequant_w4(packed, scale, zero, group), bias).reshape(*lead, -1)


def int8_linear(x, w_q, w_scale, bias=None, input_scale=None, out_dtype=torch.bfloat16):
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x.is_cuda:
        from .quant_cuda import int8_linear_cuda
        return int8_linear_cuda(x2, w_q, w_scale, bias, input_scale, out_dtype).reshape(*lead, -1)
    if input_scale is None:
        q, s = _rb.quant_int8_per_token(x2)
    else:
        q, s = _rb.quant_int8_static(x2, input_scale.float()), input_scale.float().reshape(1, 1)
    return _rb.int8_scaled_mm(q, s, w_q, w_scale.reshape(-1), bias, out_dtype).reshape(*lead, -1)


# ----------------------------------------------------------------------------- MoE

def router_gemm(x, weight, bias=None):
    """Router logits ``x @ W.T (+ b)``.  CUDA, decode-sized batches: a CUDA-core kernel with fp32 output (the
    tensor-core GEMM's fixed cost dominates at this size); otherwise the ordinary linear."""
    if x.is_cuda and x.dim() == 2 and x.shape[0] <= 64 and weight.shape[0] <= 1024 and weight.dtype == x.dtype:
        return _c().router_gemm_small(x if x.stride(-1) == 1 else x.contiguous(), weight, bias)
    return linear(x, weight, bias)


def router_and_route(x, weight, wbias, k: int, scoring: str = "softmax", renormalize: bool = True, bias=None,
                     n_group: int = 1, topk_group: int = 1, scale: float = 1.0):
    """Router logits and top-k routing from the hidden states.  CUDA, decode-sized batches with a SMALL router
    (at most 64 K weights): one launch, logits stay in shared memory.  Larger routers keep two kernels: one CTA per
    token cannot pull a 128 x 2048 router through a single SM fast enough (measured: Qwen3-30B-A3B decode step
    8.69 ms with two kernels, 9.79 ms fused), while the GEMM kernel spreads a token over E / 32 CTAs."""
    if (x.is_cuda and x.dim() == 2 and 0 < x.shape[0] <= 64 and weight.numel() <= (64 << 10) and weight.dtype == x.dtype
            and x.shape[1] * x.element_size() + weight.shape[0] * 4 <= 90 * 1024):
        from .moe_cuda import _MODES
        w, ids = _c().router_route_small(x if x.stride(-1) == 1 else x.contiguous(), weight, wbias,
                                         None if bias is None else bias.float(), k, _MODES[scoring], renormalize,
                                         n_group, topk_group, scale)
        return w, ids
    return moe_route(router_gemm(x, weight, wbias), k, scoring, renormalize, bias, n_group, topk_group, scale)


def moe_route(logits, k: int, scoring: str = "softmax", renormalize: bool = True, bias=None, n_group: int = 1,
              topk_group: int = 1, scale: float = 1.0):
    """Router: ``(weights [T, k] fp32, ids [T, k] int32)``.

    ``softmax`` = softmax -> top-k (-> renormalise) (``_C::moe_softmax_topk(_norm)``);
    ``sigmoid`` = DeepSeek-V3 group-limited routing with a selection bias
    (``_C::moe_sigmoid_group_topk_norm``); ``softmax_after_topk`` = GPT-OSS."""
    if logits.is_cuda:
        from .moe_cuda import moe_route_cuda
        return moe_route_cuda(logits, k, scoring, renormalize, bias, n_group, topk_group, scale)
    if scoring == "softmax":
        w, ids = _rm.route_softmax_topk(logits, k, renormalize)
        return w * scale, ids
    if scoring == "softmax_after_topk":
        return _rm.route_topk_then_softmax(logits, k)
    return _rm.route_sigmoid_group_topk(logits, bias, k, n_group, topk_group, renormalize, scale)


def fused_moe(x, w13, w2, topk_weights, topk_ids, act: str = "silu", b13=None, b2=None, w13_scale=None,
              w2_scale=None, block=(128, 128), expert_map=None, num_local_experts=None):
    """Routed experts: permute -> grouped GEMM(w13) -> act*mul -> grouped GEMM(w2) -> weighted un-permute.
    ``expert_map`` (global id -> local id or -1) restricts the work to this rank's experts."""
    if x.is_cuda:
        from .moe_cuda import fused_moe_cuda
        return fused_moe_cuda(x, w13, w2, topk_weights, topk_ids, act, b13, b2, w13_scale, w2_scale, block,
                              expert_map)
    return _rm.fused_moe(x, w13, w2, topk_weights, topk_ids, act, b13, b2, w13_scale, w2_scale, block, expert_map)


# ----------------------------------------------------------------------------- MLA / sparse MLA / indexer

def bmm_heads(x, w):
    """Per-head batched product ``out[t, n, :] = x[t, n, :] @ w[n]`` - the MLA absorption BMMs
    (``torch.bmm`` with ``W_UK_T`` / ``W_UV`` in ``mla/common.py:1140-1192,2009``)."""
    if x.is_cuda:
        from .mla_cuda import bmm_heads_cuda
        return bmm_heads_cuda(x, w)
    return torch.einsum("tnk,nkd->tnd", x.float(), w.float()).to(x.dtype)


def mla_attention(q, kv_cache, block_tables, seq_lens, query_start_loc, scale: float, kv_lora_rank: int,
                  max_query_len: int, max_seq_len: int, seq_lens_cpu=None, query_start_loc_cpu=None, workspace=None,
                  return_lse: bool = False, stable_metadata: bool = False):
    """Weight-absorbed MLA attention over the latent cache (decode, spec-verify and causal prefill):
    ``q [T, N, 576]`` -> ``out [T, N, 512]`` (and the natural-log LSE ``[T, N]`` when asked; rows without any
    visible key give zeros and ``-inf``)."""
    if q.is_cuda:
        from .mla_cuda import mla_attention_cuda
        return mla_attention_cuda(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, kv_lora_rank,
                                  max_query_len, max_seq_len, workspace, return_lse=return_lse,
                                  stable_metadata=stable_metadata)
    sl = seq_lens if seq_lens_cpu is None else seq_lens_cpu
    ql = query_start_loc if query_start_loc_cpu is None else query_start_loc_cpu
    return _ra.mla_decode(q, kv_cache, block_tables, sl, ql, scale, kv_lora_rank, return_lse=return_lse)


def mla_prefill_attention(q, kv, k_pe, kv_starts, kv_lens, query_start_loc, causal: bool, scale: float,
                          max_query_len: int, out=None, lse=None):
    """MLA prefill in the up-projected 192 / 128 form over contiguous keys (the new tokens themselves, causal; or a
    gathered and up-projected chunk of cached context, not causal): ``q [T, N, 192]``, ``kv [rows, N * 256]``,
    ``k_pe [rows, 64]`` -> ``out [T, N, 128]``, natural-log ``lse [T, N]``.  Rows of requests without keys give
    zeros and ``-inf``.  CUDA: the tcgen05 prefill kernel (``csrc/attention/prefill_umma.cu``, MLA instantiation)."""
    if q.is_cuda:
        T, N, _ = q.shape
        if out is None:
            out = torch.zeros(T, N, 128, dtype=q.dtype, device=q.device)
        if lse is None:
            lse = torch.full((T, N), float("-inf"), dtype=torch.float32, device=q.device)
        _c().mla_prefill_umma(out, q, kv, k_pe, kv_starts, kv_lens, query_start_loc, lse, int(max_query_len),
                              bool(causal), float(scale))
        return out, lse
    return _ra.mla_prefill(q, kv, k_pe, kv_starts, kv_lens, query_start_loc, causal, scale)


def sparse_mla_attention(q, kv_cache, indices, scale: float, d_v: int = 512):
    """DeepSeek sparse attention: every query row attends its own ``indices [T, topk]`` (global slot ids,
    -1 = none) of the flat latent cache.  Returns ``out [T, N, d_v]``."""
    flat = kv_cache.reshape(-1, kv_cache.shape[-1])
    if q.is_cuda:
        from .mla_cuda import sparse_mla_cuda
        return sparse_mla_cuda(q, flat, indices, scale, d_v)
    return _ra.sparse_mla(q, flat, indices, scale, d_v)[0]


def indexer_topk(q_fp8, q_scale, weights, k_cache, block_tables, seq_lens, query_start_loc, topk: int,
                 seq_lens_cpu=None, query_start_loc_cpu=None):
    """Lightning-indexer scores over the paged fp8 key cache and per-row top-k.

    ``q_fp8 [T, H, 128]`` (e4m3) with per-(token, head) ``q_scale [T, H]``; ``weights [T, H]``.  Row ``t`` of
    request ``r`` sits at position ``p`` and scores keys ``0..p``.  Returns request-local token indices
    ``[T, topk]`` (int32, -1 padded): ``_C::I8_(paged_)mqa_logits`` + ``topk_per_row`` of the reference
    (``models/deepseek_v2.py:527-637``) in one call."""
    if q_fp8.is_cuda:
        from .mla_cuda import indexer_topk_cuda
        return indexer_topk_cuda(q_fp8, q_scale, weights, k_cache, block_tables, seq_lens, query_start_loc, topk)
    sl = seq_lens if seq_lens_cpu is None else seq_lens_cpu
    ql = query_start_loc if query_start_loc_cpu is None else query_start_loc_cpu
    T = q_fp8.shape[0]
    out = torch.full((T, topk), -1, dtype=torch.int32)
    bs = k_cache.shape[1]
    qf = q_fp8.float() * q_scale.float().unsqueeze(-1)
    for r in range(block_tables.shape[0]):
        qs, qe = int(ql[r]), int(ql[r + 1])
        if qe == qs:
            continue
        L = int(sl[r])
        pos = torch.arange(L)
        kv, sv = _ra.indexer_cache_views(k_cache)
        blk = block_tables[r, pos // bs].long()
        k = kv[blk, pos % bs].contiguous().view(torch.float8_e4m3fn).float()
        ksc = sv[blk, pos % bs].reshape(-1)
        n = qe - qs
        ke = torch.arange(L - n + 1, L + 1)
        logits = _ra.indexer_logits(qf[qs:qe], k, ksc, weights[qs:qe], torch.zeros(n, dtype=torch.long), ke)
        out[qs:qe] = _ra.topk_per_row(logits, torch.zeros(n, dtype=torch.long), ke, topk)
    return out


# ----------------------------------------------------------------------------- sampling kernels

_sample_step = [0]
_seen_bitmaps: dict = {}


def topk_topp_sample(logits, temperature=None, top_k=None, top_p=None, noise=None, seed: int = 0):
    """Temperature / top-k / top-p / exponential-race draw, one launch for the whole batch.
    ``temperature == 0`` rows are greedy.  ``noise [B, V]`` (Exp(1) variates) overrides the in-kernel
    counter-based generator."""
    if logits.is_cuda:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
        _sample_step[0] += 1
        _c().topk_topp_sample(out, logits, temperature, None if top_k is None else top_k.int(), top_p, noise, seed,
                              _sample_step[0])
        return out
    B = logits.shape[0]
    t = temperature if temperature is not None else torch.ones(B)
    return _rx.sample(logits, t, top_k, top_p, q=noise)


def apply_repetition_penalty(logits, token_ids, num_tokens, penalties):
    """In place: for every distinct token of ``token_ids[b, :num_tokens[b]]``, positive logits are divided by
    the row's penalty and negative ones multiplied (``apply_repetition_penalties_`` of the reference)."""
    if logits.is_cuda:
        B, V = logits.shape
        key = (logits.device, B, V)
        seen = _seen_bitmaps.get(key)
        if seen is None:
            seen = _seen_bitmaps[key] = torch.empty(B * ((V + 31) // 32), dtype=torch.int32, device=logits.device)
        _c().repetition_penalty(logits, token_ids, num_tokens.int(), penalties.float(), seen)
        return logits
    for b in range(logits.shape[0]):
        ids = token_ids[b, : int(num_tokens[b])].unique()
        ids = ids[(ids >= 0) & (ids < logits.shape[1])]
        row = logits[b, ids].float()
        pen = float(penalties[b])
        logits[b, ids] = torch.where(row > 0, row / pen, row * pen).to(logits.dtype)
    return logits


def rejection_sample(draft_token_ids, num_draft, target_probs, bonus_token_ids, is_greedy, draft_probs=None,
                     uniform=None, recover_q=None, max_spec_len: int = 1, seed: int = 0):
    """Speculative-decoding verifier, one block per request; output ``[B, max_spec_len + 1]`` padded with -1."""
    B = num_draft.shape[0]
    if target_probs.is_cuda:
        out = torch.empty(B, max_spec_len + 1, dtype=torch.int64, device=target_probs.device)
        cu = torch.zeros(B + 1, dtype=torch.int32, device=target_probs.device)
        cu[1:] = num_draft.cumsum(0)
        _sample_step[0] += 1
        _c().rejection_sample(out, draft_token_ids.long(), cu, target_probs.float().contiguous(),
                              None if draft_probs is None else draft_probs.float().contiguous(), bonus_token_ids.long(),
                              is_greedy.to(torch.uint8), uniform, recover_q, seed, _sample_step[0])
        return out
    from ..sample.rejection_sampler import RejectionSampler
    return RejectionSampler().forward(draft_token_ids, num_draft, target_probs, bonus_token_ids, is_greedy, draft_probs,
                                      uniform, recover_q, max_spec_len)


# ----------------------------------------------------------------------------- conv / gated delta net

def causal_conv1d_fn(x, weight, bias, cu_seqlens, conv_states, state_indices, has_initial_state, activation=True):
    if x.is_cuda:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        _c().causal_conv1d_fwd(out, x, weight, bias, cu_seqlens.int(), conv_states, state_indices.int(),
                               has_initial_state.to(torch.uint8), activation)
        return out
    return _rx.causal_conv1d_fn(x, weight, bias, cu_seqlens, conv_states, state_indices, has_initial_state, activation)


def causal_conv1d_update(x, conv_states, weight, bias, state_indices, activation=True):
    if x.is_cuda:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        _c().causal_conv1d_update(out, x, conv_states, weight, bias, state_indices.int(), activation)
        return out
    return _rx.causal_conv1d_update(x, conv_states, weight, bias, state_indices, activation)


def fused_gdn_gating(A_log, a, b, dt_bias):
    """``g = -exp(A_log) * softplus(a + dt_bias)``, ``beta = sigmoid(b)``; fp32 ``[T, Hv]`` each."""
    if a.is_cuda:
        g = torch.empty(a.shape, dtype=torch.float32, device=a.device)
        beta = torch.empty_like(g)
        _c().gdn_gating(g, beta, a, b, A_log.float(), dt_bias.float())
        return g, beta
    g = -torch.exp(A_log.float()) * torch.nn.functional.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


GDN_CHUNK_MIN = 64      # new tokens of a request from which the chunked form is used (when it is enabled)


def gated_delta_rule(q, k, v, g, beta, states, cu_seqlens, state_indices, has_initial_state, scale=None,
                     use_qk_l2norm=True, cu_seqlens_cpu=None):
    """Varlen gated delta rule over a state cache ``[slots, Hv, Dv, Dk]`` (fp32, updated in place).
    ``q, k [T, Hk, Dk]``, ``v [T, Hv, Dv]``, ``g, beta [T, Hv]`` fp32.  Serves prefill and decode alike with the
    recurrent kernel (one dependent step per token).  With ``B200_GDN_CHUNKED=1`` and the host copy of the segment
    offsets, requests with at least ``GDN_CHUNK_MIN`` new tokens take the chunked form instead (the reference's
    prefill path, ``ops/fla/chunk.py:23-140``): batched matrix products per 64-token chunk and one state update per
    chunk; the other requests of the step keep the recurrent kernel."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    long_rows = []
    if cu_seqlens_cpu is not None:
        from .. import envs
        if envs.B200_GDN_CHUNKED:
            lens = (cu_seqlens_cpu[1:] - cu_seqlens_cpu[:-1]).tolist()
            long_rows = [r for r, n in enumerate(lens) if n >= GDN_CHUNK_MIN]
    out = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    slots = state_indices
    if long_rows:
        rows_t = torch.tensor(long_rows, dtype=torch.long).to(v.device, non_blocking=True)
        slots = state_indices.clone()
        slots[rows_t] = -1          # the recurrent pass skips them
    if len(long_rows) < len(cu_seqlens) - 1:
        if q.is_cuda:
            _c().gdn_recurrent(out, q, k, v, g, beta, states, cu_seqlens.int(), slots.int(),
                               has_initial_state.to(torch.uint8), scale, use_qk_l2norm)
        else:
            for r in range(len(cu_seqlens) - 1):
                s, e = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
                slot = int(slots[r])
                if e == s or slot < 0:
                    continue
                S0 = states[slot] if bool(has_initial_state[r]) else torch.zeros_like(states[slot])
                o, S = _rx.recurrent_gated_delta_rule(q[s:e], k[s:e], v[s:e], g[s:e], beta[s:e], S0, scale, use_qk_l2norm)
                out[s:e] = o
                states[slot] = S
    for r in long_rows:             # offsets from the host copy; slot and initial-state flag stay on the device
        s, e = int(cu_seqlens_cpu[r]), int(cu_seqlens_cpu[r + 1])
        slot = state_indices[r].view(1).long()
        S0 = states.index_select(0, slot)[0] * has_initial_state[r].to(states.dtype)
        o, S = _rx.chunk_gated_delta_rule_batched(q[s:e], k[s:e], v[s:e], g[s:e], beta[s:e], S0, 64, scale, use_qk_l2norm)
        out[s:e] = o
        states.index_copy_(0, slot, S.unsqueeze(0).to(states.dtype))
    return out


def sigmoid_gate_mul(o, gate):
    """``o * sigmoid(gate)``; ``gate`` may be a column slice of a wider tensor."""
    if o.is_cuda:
        out = torch.empty(o.shape, dtype=o.dtype, device=o.device)
        _c().sigmoid_gate_mul(out, o.contiguous(), gate)
        return out
    return (o.float() * torch.sigmoid(gate.float())).to(o.dtype)


def mtp_concat_norm(embed, hidden, enorm_w, hnorm_w, eps, positions=None):
    """MTP layer input: ``[rmsnorm(embed) (zeroed at position 0), rmsnorm(hidden)]`` (``deepseek_mtp.py:79-87``)."""
    if embed.is_cuda:
        out = torch.empty(embed.shape[0], 2 * embed.shape[1], dtype=embed.dtype, device=embed.device)
        _c().mtp_concat_norm(out, embed.contiguous(), hidden.contiguous(), enorm_w, hnorm_w, positions, eps)
        return out
    e = embed if positions is None else torch.where((positions == 0).unsqueeze(-1), torch.zeros_like(embed), embed)
    return torch.cat([_rb.rmsnorm(e, enorm_w, eps), _rb.rmsnorm(hidden, hnorm_w, eps)], -1)


# ----------------------------------------------------------------------------- LoRA

def lora_shrink(x, lora_a, token_lora_ids, scale: float = 1.0):
    """``out[t] = x[t] @ A[id[t]].T * scale`` (fp32 ``[T, r]``); ``id < 0`` rows are zero."""
    if x.is_cuda:
        out = torch.empty(x.shape[0], lora_a.shape[1], dtype=torch.float32, device=x.device)
        _c().lora_shrink(out, x, lora_a, token_lora_ids.int(), scale)
        return out
    return _rx.bgmv_shrink(x, lora_a, token_lora_ids, scale)


def lora_expand(h, lora_b, token_lora_ids, out, offset: int = 0, add: bool = True):
    """``out[t, offset:offset+N] (+)= h[t] @ B[id[t]].T``."""
    if out.is_cuda:
        _c().lora_expand(out, h, lora_b, token_lora_ids.int(), offset, add)
        return out
    return _rx.bgmv_expand(h, lora_b, token_lora_ids, out, offset, add)


__all__ = [n for n in dir() if not n.startswith("_")]


# ----------------------------------------------------------------------------- vision-tower ops

_SUPPORTED_HEAD_DIMS = (64, 128, 256)


def varlen_attention(q, k, v, cu_seqlens, scale: Optional[float] = None, max_seqlen: Optional[int] = None):
    """Bidirectional attention over packed sequences (ViT blocks; the reference calls
    ``flash_attn_varlen_func`` / SDPA, ``models/qwen2_5_vl.py:356-393``, ``ops/attention/layer.py:121-180``).
    ``q, k, v [T, H, D]``.  CUDA: K/V are laid out as pages of a scratch cache and the prefill kernel runs in
    its bidirectional mode; head sizes are zero-padded to the next supported size (exact)."""
    T, H, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    if not q.is_cuda:
        out = torch.empty_like(q)
        for i in range(len(cu_seqlens) - 1):
            s, e = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
            if e > s:
                out[s:e] = _ra._attend(q[s:e], k[s:e], v[s:e], scale, None, None, None).to(q.dtype)
        return out
    Dp = next(d for d in _SUPPORTED_HEAD_DIMS if d >= D)
    if Dp != D:
        pad = (0, Dp - D)
        q, k, v = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
    bs = 64
    cu = cu_seqlens.to(torch.int64)
    lens = cu[1:] - cu[:-1]
    nblk = (lens + bs - 1) // bs
    first = torch.zeros_like(nblk)
    first[1:] = nblk.cumsum(0)[:-1]
    total_blocks = int(nblk.sum().item())
    max_blocks = int(nblk.max().item())
    tok = torch.arange(T, device=q.device)
    seq_of = torch.searchsorted(cu[1:], tok, right=True)
    slots = first[seq_of] * bs + (tok - cu[seq_of])
    cache = torch.empty(total_blocks, 2, H, bs, Dp, dtype=q.dtype, device=q.device)
    _c().reshape_and_cache(k.contiguous(), v.contiguous(), cache, slots)
    bt = (first.unsqueeze(1) + torch.arange(max_blocks, device=q.device).unsqueeze(0)).clamp(max=total_blocks - 1).int()
    out = torch.empty(T, H, Dp, dtype=q.dtype, device=q.device)
    mq = int(lens.max().item()) if max_seqlen is None else max_seqlen
    _c().paged_attention(out, q.contiguous(), cache, bt.contiguous(), lens.int(), cu.int(), None, None, None, max(mq, 17), 1,
                         -1, scale, False)
    return out[..., :D] if Dp != D else out


def rope_vit(q, k, cos, sin):
    """2-D rotary embedding of vision tokens (``xspeedgate_ops.rope_vit``, ``models/qwen2_vl.py:255``):
    rotate-half with per-token ``cos / sin [T, D/2]`` shared by all heads."""
    def rot(x):
        xf = x.float()
        d = xf.shape[-1] // 2
        c, s = cos.float().unsqueeze(1), sin.float().unsqueeze(1)
        x1, x2 = xf[..., :d], xf[..., d:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)
    return rot(q), rot(k)


def layernorm(x, weight, bias, eps: float):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(),
                                          eps).to(x.dtype)


__all__ = [n for n in dir() if not n.startswith("_")]
