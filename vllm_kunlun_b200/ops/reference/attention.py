"""fp32 PyTorch oracles: KV-cache movement, paged GQA attention, MLA, sparse MLA, indexer.

Cache layouts of this framework (chosen so a page of one KV head is one contiguous,
16-byte-aligned run that a bulk copy or a TMA box can fetch):

* GQA:  ``kv_cache[num_blocks, 2, num_kv_heads, block_size, head_dim]``
  (the reference keeps ``(2, blocks, kv_heads, block_size, head)``, ``ops/paged_attn.py:43-55``)
* MLA:  ``kv_cache[num_blocks, block_size, 576]`` = ``[kv_c(512) | k_pe(64)]``
  (``v1/attention/backends/mla/common.py:296-304``)
* fp8_ds_mla: ``uint8[num_blocks, block_size, 656]`` = 512 e4m3 | 4 fp32 scales | 64 bf16 rope
  (``v1/attention/backends/mla/flashmla_sparse.py:357-425``)
* indexer K: ``uint8[num_blocks, block_size, 132]`` holding, per block, ``block_size`` rows of 128 e4m3 bytes and
  then ``block_size`` fp32 scales (page-major: a page's key rows are one contiguous, 16-byte aligned tile)
  (``models/deepseek_v2.py:714-719``)
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .basic import FP8_MAX


# ----------------------------------------------------------------------------- cache writes

def reshape_and_cache(k, v, kv_cache, slot_mapping):
    """``kunlun_ops.reshape_and_cache_flash`` (``v1/attention/backends/kunlun_attn.py:805-812``).
    ``k, v [T, Hkv, D]``; slots < 0 are skipped (padding)."""
    bs = kv_cache.shape[3]
    for t in range(k.shape[0]):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        kv_cache[s // bs, 0, :, s % bs] = k[t].to(kv_cache.dtype)
        kv_cache[s // bs, 1, :, s % bs] = v[t].to(kv_cache.dtype)


def concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping):
    """``_C::concat_and_cache_mla`` bf16 layout (``ops/_custom_ops.py:1588-1616``)."""
    bs = kv_cache.shape[1]
    for t in range(kv_c.shape[0]):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        kv_cache[s // bs, s % bs, : kv_c.shape[1]] = kv_c[t].to(kv_cache.dtype)
        kv_cache[s // bs, s % bs, kv_c.shape[1]:] = k_pe[t].to(kv_cache.dtype)


def concat_and_cache_mla_fp8(kv_c, k_pe, kv_cache_u8, slot_mapping):
    """656-byte ``fp8_ds_mla`` packing: 4 groups of 128 e4m3 values with one fp32 scale each,
    followed by the 64 rope values in bf16 (python reference at ``flashmla_sparse.py:357-425``)."""
    bs = kv_cache_u8.shape[1]
    for t in range(kv_c.shape[0]):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        row = kv_cache_u8[s // bs, s % bs]
        g = kv_c[t].float().reshape(4, 128)
        scale = g.abs().amax(-1).clamp(min=1e-10) / FP8_MAX
        q = (g / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
        row[:512] = q.reshape(-1).view(torch.uint8)
        row[512:528] = scale.to(torch.float32).view(torch.uint8)
        row[528:656] = k_pe[t].to(torch.bfloat16).view(torch.uint8)


def dequant_mla_fp8_rows(rows_u8: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`concat_and_cache_mla_fp8` for ``[..., 656]`` rows -> ``[..., 576]`` fp32."""
    lead = rows_u8.shape[:-1]
    r = rows_u8.reshape(-1, 656)
    q = r[:, :512].contiguous().view(torch.float8_e4m3fn).float().reshape(-1, 4, 128)
    sc = r[:, 512:528].contiguous().view(torch.float32).reshape(-1, 4, 1)
    pe = r[:, 528:656].contiguous().view(torch.bfloat16).float()
    return torch.cat([(q * sc).reshape(-1, 512), pe], -1).reshape(*lead, 576)


def indexer_k_quant_and_cache(k, k_cache_u8, slot_mapping, ue8m0: bool = True):
    """``xspeedgate_ops.indexer_k_quant_and_cache`` (``models/deepseek_v2.py:519-525``):
    one 128-wide group per token, e4m3 payload + fp32 scale (power of two when ``ue8m0``)."""
    bs = k_cache_u8.shape[1]
    for t in range(k.shape[0]):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        kf = k[t].float()
        scale = kf.abs().amax().clamp(min=1e-10) / FP8_MAX
        if ue8m0:
            scale = torch.exp2(torch.ceil(torch.log2(scale)))
        q = (kf / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
        kv, sv = indexer_cache_views(k_cache_u8)
        kv[s // bs, s % bs] = q.view(torch.uint8)
        sv[s // bs, s % bs] = scale.to(torch.float32)


def indexer_cache_views(k_cache_u8):
    """``(keys uint8 [blocks, block_size, 128], scales float32 [blocks, block_size])`` views of the indexer cache:
    per block, the key rows come first and the scales after them."""
    nb, bs, w = k_cache_u8.shape
    assert w == 132
    flat = k_cache_u8.view(nb, bs * 132)
    return flat[:, : bs * 128].view(nb, bs, 128), flat[:, bs * 128:].view(torch.float32)


def gather_indexer_k(k_cache_u8, block_table, cu_seq_lens):
    """``cp_gather_indexer_k_quant_cache`` (``models/deepseek_v2.py:536-542``): paged -> contiguous
    ``(k_fp8 [sum, 128], scale [sum])``."""
    bs = k_cache_u8.shape[1]
    outs_k, outs_s = [], []
    for r in range(block_table.shape[0]):
        n = int(cu_seq_lens[r + 1] - cu_seq_lens[r])
        pos = torch.arange(n)
        kv, sv = indexer_cache_views(k_cache_u8)
        blk = block_table[r, pos // bs].long()
        outs_k.append(kv[blk, pos % bs].contiguous().view(torch.float8_e4m3fn))
        outs_s.append(sv[blk, pos % bs].reshape(-1))
    return torch.cat(outs_k), torch.cat(outs_s)


def gather_mla_cache(kv_cache, block_table, cu_seq_lens, seq_starts=None):
    """``gather_and_maybe_dequant_cache`` (``mla/common.py:1557-1612``): rows of a context chunk."""
    bs = kv_cache.shape[1]
    outs = []
    for r in range(block_table.shape[0]):
        n = int(cu_seq_lens[r + 1] - cu_seq_lens[r])
        st = 0 if seq_starts is None else int(seq_starts[r])
        pos = torch.arange(st, st + n)
        rows = kv_cache[block_table[r, pos // bs].long(), pos % bs]
        if kv_cache.dtype == torch.uint8:
            rows = dequant_mla_fp8_rows(rows)
        outs.append(rows)
    return torch.cat(outs)


def convert_req_index_to_global_index(req_id, block_table, token_indices, block_size: int):
    """``convert_req_index_to_global_index`` (torch reference ``flashmla_sparse.py:305-354``):
    ``out[t, j] = block_table[req[t], idx // bs] * bs + idx % bs``, ``-1`` preserved."""
    idx = token_indices.long()
    valid = idx >= 0
    safe = idx.clamp(min=0)
    blk = safe // block_size
    in_range = blk < block_table.shape[1]
    blk = blk.clamp(max=block_table.shape[1] - 1)
    base = torch.gather(block_table[req_id.long()].long(), 1, blk)
    out = base * block_size + safe % block_size
    return torch.where(valid & in_range, out, torch.full_like(out, -1)).to(torch.int32)


def swap_blocks(src, dst, mapping):
    for s, d in mapping:
        dst[d].copy_(src[s])


def copy_blocks(caches, mapping):
    for c in caches:
        for s, d in mapping:
            c[d].copy_(c[s])


# ----------------------------------------------------------------------------- GQA attention

def _attend(q, k, v, scale, causal_offset: Optional[int], window: Optional[int], sinks, return_lse=False,
            softcap: float = 0.0):
    """q [Lq, Hq, D], k/v [Lk, Hkv, D(v)].  Query row i sits at absolute position
    ``causal_offset + i`` and sees keys ``<=`` that position (None = no mask)."""
    Lq, Hq, D = q.shape
    Lk, Hkv = k.shape[0], k.shape[1]
    g = Hq // Hkv
    qf = q.float().reshape(Lq, Hkv, g, D).permute(1, 2, 0, 3)  # [Hkv,g,Lq,D]
    kf = k.float().permute(1, 0, 2).unsqueeze(1)  # [Hkv,1,Lk,D]
    vf = v.float().permute(1, 0, 2).unsqueeze(1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale  # [Hkv,g,Lq,Lk]
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    if causal_offset is not None:
        qpos = torch.arange(Lq).unsqueeze(1) + causal_offset
        kpos = torch.arange(Lk).unsqueeze(0)
        mask = kpos <= qpos
        if window is not None:
            mask &= kpos > qpos - window
        s = s.masked_fill(~mask, float("-inf"))
    m = s.amax(-1, keepdim=True)
    if sinks is not None:
        sk = sinks.float().reshape(Hkv, g, 1, 1)
        m = torch.maximum(m, sk)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m)
    denom = p.sum(-1, keepdim=True)
    if sinks is not None:
        denom = denom + torch.exp(sk - m)
    o = torch.matmul(p, vf) / denom.clamp(min=1e-30)
    o = o.permute(2, 0, 1, 3).reshape(Lq, Hq, -1)
    if return_lse:
        lse = (m + torch.log(denom.clamp(min=1e-30))).squeeze(-1).permute(2, 0, 1).reshape(Lq, Hq)
        return o, lse
    return o


def gather_paged_kv(kv_cache, block_table_row, seq_len: int):
    bs = kv_cache.shape[3]
    pos = torch.arange(seq_len)
    blk = block_table_row[pos // bs].long()
    k = kv_cache[blk, 0, :, pos % bs]  # [L, Hkv, D]
    v = kv_cache[blk, 1, :, pos % bs]
    return k, v


def paged_attention(q, kv_cache, block_tables, seq_lens, query_start_loc, scale,
                    window: Optional[int] = None, sinks=None, softcap: float = 0.0):
    """Unified varlen paged attention: covers ``kunlun_ops.prefill_attention`` (with prefix cache,
    ``kunlun_attn.py:849-891``) and ``kunlun_ops.speculative_attention`` (decode with
    ``q_len >= 1``, ``kunlun_attn.py:926-947``).  K/V for all ``seq_lens[r]`` positions are read
    from the cache; the ``q_len`` queries of request ``r`` are its last positions."""
    out = torch.empty(q.shape[0], q.shape[1], kv_cache.shape[-1], dtype=q.dtype)
    for r in range(block_tables.shape[0]):
        qs, qe = int(query_start_loc[r]), int(query_start_loc[r + 1])
        if qe == qs:
            continue
        L = int(seq_lens[r])
        k, v = gather_paged_kv(kv_cache, block_tables[r], L)
        out[qs:qe] = _attend(q[qs:qe], k, v, scale, L - (qe - qs), window, sinks, softcap=softcap).to(q.dtype)
    return out


def varlen_attention(q, k, v, cu_q, cu_k, scale, causal=True, return_lse=False, window=None, sinks=None):
    """``kunlun_ops.attention`` (``mla/common.py:1286-1305``): dense varlen MHA with optional LSE and
    different QK / V head dims."""
    out = torch.empty(q.shape[0], q.shape[1], v.shape[-1], dtype=q.dtype)
    lse = torch.empty(q.shape[0], q.shape[1], dtype=torch.float32)
    for r in range(len(cu_q) - 1):
        qs, qe, ks, ke = int(cu_q[r]), int(cu_q[r + 1]), int(cu_k[r]), int(cu_k[r + 1])
        if qe == qs:
            continue
        off = (ke - ks) - (qe - qs) if causal else None
        if ke == ks:
            out[qs:qe] = 0
            lse[qs:qe] = float("-inf")
            continue
        o, l = _attend(q[qs:qe], k[ks:ke], v[ks:ke], scale, off, window, sinks, return_lse=True)
        out[qs:qe], lse[qs:qe] = o.to(q.dtype), l
    return (out, lse) if return_lse else out


def merge_attn_states(o1, lse1, o2, lse2):
    """``kunlun_ops.attention_merge_stage`` (``ops/attention/merge_attn_states.py:18-20``).
    ``o [T, H, D]``, ``lse [T, H]`` (natural log)."""
    m = torch.maximum(lse1, lse2)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    den = (w1 + w2).clamp(min=1e-30)
    o = (o1.float() * w1.unsqueeze(-1) + o2.float() * w2.unsqueeze(-1)) / den.unsqueeze(-1)
    return o.to(o1.dtype), m + torch.log(den)


# ----------------------------------------------------------------------------- MLA

def mla_prefill(q, kv, k_pe, kv_starts, kv_lens, query_start_loc, causal: bool, scale: float):
    """Multi-head latent attention in the up-projected ("compute-friendly") form used for prefill
    (``v1/attention/backends/mla/common.py:1782-1843``): ``q [T, N, 192]`` (q_nope | rotated q_pe),
    ``kv [rows, N * 256]`` (k_nope | v per head: the ``kv_b_proj`` output), ``k_pe [rows, 64]`` (one rotary key per
    token, shared by the heads).  Request ``r`` owns key rows ``kv_starts[r] .. + kv_lens[r]`` and query rows
    ``query_start_loc[r] .. [r + 1]``; causal: its queries are its last keys; otherwise every query sees every key
    (a chunk of cached context).  Returns ``out [T, N, 128]`` and the natural-log LSE ``[T, N]``; rows of requests
    without keys give zeros and ``-inf``."""
    T, N, dq = q.shape
    nope = dq - k_pe.shape[1]                       # 128 in the checkpoints; the oracle takes any split
    vdim = kv.shape[1] // N - nope
    out = torch.zeros(T, N, vdim, dtype=q.dtype)
    lse = torch.full((T, N), float("-inf"))
    kvh = kv.reshape(kv.shape[0], N, nope + vdim).float()
    for r in range(len(kv_lens)):
        qs, qe = int(query_start_loc[r]), int(query_start_loc[r + 1])
        ks, L = int(kv_starts[r]), int(kv_lens[r])
        if qe == qs or L == 0:
            continue
        k = torch.cat([kvh[ks:ks + L, :, :nope], k_pe[ks:ks + L].float().unsqueeze(1).expand(-1, N, -1)], -1)
        v = kvh[ks:ks + L, :, nope:]
        s = torch.einsum("qnd,knd->nqk", q[qs:qe].float(), k) * scale
        if causal:
            pos = (L - (qe - qs)) + torch.arange(qe - qs)
            s = s.masked_fill(torch.arange(L)[None, None, :] > pos[None, :, None], float("-inf"))
        l = torch.logsumexp(s, -1)                                   # [N, q]
        p = torch.exp(s - l.unsqueeze(-1))
        out[qs:qe] = torch.einsum("nqk,knd->qnd", p, v).to(q.dtype)
        lse[qs:qe] = l.t()
    return out, lse


def mla_decode(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, kv_lora_rank: int = 512,
               return_lse: bool = False):
    """Weight-absorbed MQA decode (``flash_mla_with_kvcache``, ``ops/attention/flashmla.py:61-128``).
    ``q [T, N, 576]`` (``[q_nope . W_UK | q_pe]``), cache ``[blocks, bs, 576]`` (or 656-byte fp8).
    Output ``[T, N, 512]``; the ``q_len`` rows of a request are its last positions (causal)."""
    T, N, _ = q.shape
    out = torch.zeros(T, N, kv_lora_rank, dtype=q.dtype)
    lse = torch.full((T, N), float("-inf"))
    bs = kv_cache.shape[1]
    for r in range(block_tables.shape[0]):
        qs, qe = int(query_start_loc[r]), int(query_start_loc[r + 1])
        if qe == qs:
            continue
        L = int(seq_lens[r])
        if L == 0:  # nothing cached for this row (possible on a context-parallel rank): zeros and -inf
            continue
        pos = torch.arange(L)
        rows = kv_cache[block_tables[r, pos // bs].long(), pos % bs]
        rows = dequant_mla_fp8_rows(rows) if kv_cache.dtype == torch.uint8 else rows.float()
        k = rows.unsqueeze(1)  # [L,1,576]
        v = rows[:, :kv_lora_rank].unsqueeze(1)
        o, l = _attend(q[qs:qe], k, v, scale, L - (qe - qs), None, None, return_lse=True)
        out[qs:qe], lse[qs:qe] = o.to(q.dtype), l
    return (out, lse) if return_lse else out


def sparse_mla(q, kv_flat, indices, scale, d_v: int = 512):
    """``_C::sparse_prefill_fwd_opt`` / ``_C::fwd_kvcache_mla`` (``ops/_custom_ops.py:2148-2311``).
    ``q [T, N, 576]``, ``kv_flat [slots, 576]`` (or ``[slots, 656]`` uint8), ``indices [T, topk]``
    global slot ids with ``-1`` = invalid.  Returns ``(out [T,N,d_v], max_logits [T,N], lse2 [T,N])``
    where ``lse2`` is the base-2 log-sum-exp."""
    T, N, _ = q.shape
    out = torch.zeros(T, N, d_v, dtype=q.dtype)
    mx = torch.full((T, N), float("-inf"))
    lse = torch.full((T, N), float("-inf"))
    for t in range(T):
        idx = indices[t].long()
        idx = idx[idx >= 0]
        if idx.numel() == 0:
            continue
        rows = kv_flat[idx]
        rows = dequant_mla_fp8_rows(rows) if kv_flat.dtype == torch.uint8 else rows.float()
        s = torch.einsum("nd,ld->nl", q[t].float(), rows) * scale
        m = s.amax(-1)
        p = torch.exp(s - m[:, None])
        den = p.sum(-1)
        out[t] = ((p @ rows[:, :d_v]) / den[:, None]).to(q.dtype)
        mx[t] = m
        lse[t] = (m + torch.log(den)) / math.log(2.0)
    return out, mx, lse


# ----------------------------------------------------------------------------- lightning indexer

def indexer_logits(q, k, k_scale, weights, ks, ke):
    """``_C::I8_mqa_logits`` + mask (``ops/deep_gemm.py:5-55``):
    ``logits[m, n] = sum_h w[m, h] * relu(q[m, h, :] . k[n, :]) * k_scale[n]`` for
    ``ks[m] <= n < ke[m]``, ``-inf`` elsewhere.  ``q [M, H, 128]``, ``k [N, 128]``."""
    s = torch.einsum("mhd,nd->mhn", q.float(), k.float())
    logits = (torch.relu(s) * weights.float().unsqueeze(-1)).sum(1) * k_scale.float().unsqueeze(0)
    n = torch.arange(k.shape[0]).unsqueeze(0)
    mask = (n >= ks.unsqueeze(1)) & (n < ke.unsqueeze(1))
    return logits.masked_fill(~mask, float("-inf"))


def indexer_logits_paged(q, k_cache_u8, weights, seq_lens, block_table, max_len: int):
    """``_C::I8_paged_mqa_logits`` (``ops/deep_gemm.py:58-121``).  ``q [B, next_n, H, 128]``;
    row ``b*next_n + j`` sees keys ``< seq_lens[b] - next_n + j + 1``.  Output ``[B*next_n, max_len]``."""
    B, nn_, H, D = q.shape
    bs = k_cache_u8.shape[1]
    out = torch.full((B * nn_, max_len), float("-inf"))
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        pos = torch.arange(L)
        kv, sv = indexer_cache_views(k_cache_u8)
        blk = block_table[b, pos // bs].long()
        k = kv[blk, pos % bs].contiguous().view(torch.float8_e4m3fn).float()
        sc = sv[blk, pos % bs].reshape(-1)
        for j in range(nn_):
            lim = L - nn_ + j + 1
            s = torch.einsum("hd,nd->hn", q[b, j].float(), k[:lim])
            out[b * nn_ + j, :lim] = (torch.relu(s) * weights[b * nn_ + j].float().unsqueeze(-1)).sum(0) * sc[:lim]
    return out


def topk_per_row(logits, row_starts, row_ends, k: int):
    """``xspeedgate_ops.topk_per_row`` (``models/deepseek_v2.py:563-574``): indices (relative to
    ``row_starts``) of the ``k`` largest logits in ``[start, end)``; ``-1`` pads short rows."""
    M = logits.shape[0]
    out = torch.full((M, k), -1, dtype=torch.int32)
    for m in range(M):
        s, e = int(row_starts[m]), int(row_ends[m])
        if e <= s:
            continue
        seg = logits[m, s:e].float()
        kk = min(k, e - s)
        out[m, :kk] = torch.topk(seg, kk).indices.to(torch.int32)
    return out
